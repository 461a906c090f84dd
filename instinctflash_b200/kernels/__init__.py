"""Engine kernels of the FP8 linear path (drop-in names of ``instinctflash.kernels``).

Contract kept from the reference (instinctflash/kernels/__init__.py:1-29): activations are
quantised to e4m3 per row where they are produced and the row scale travels with them;
weights carry one scale per output channel; ``gemm`` runs with unit scales and writes the raw
accumulator in bf16; the consumer applies ``row_scale[m] * col_scale[n]`` (+ bias).  Every
operator writes into caller-owned tensors on the current CUDA stream, allocates nothing and
is CUDA-graph capturable.

Importing this package needs neither a GPU nor the shared library; calling an operator does.
"""
