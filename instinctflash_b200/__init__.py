"""B200-native (sm_100a) FP8 linear path behind the InstinctFlash engine-kernel signatures.

Per-token e4m3 activation quantisation, the tcgen05 FP8 GEMM and its fused bias / gated /
residual consumers, as hand-written CUDA in ``libiflb200.so`` (C ABI in ``include/iflb200.h``).
``instinctflash_b200.kernels`` mirrors the operator names and signatures of
``instinctflash.kernels.{fp8,norm,activation}``; ``instinctflash_b200.runtime`` mirrors the
per-tensor recipe of ``instinctflash.runtime.{fp8_pack,torch_fp8_linear}``.
"""
__version__ = "0.1.0"
