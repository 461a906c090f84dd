"""Per-tensor FP8 projections (drop-in names of ``instinctflash.runtime.fp8_pack`` and
``instinctflash.runtime.torch_fp8_linear``) on the sm_100a kernels."""
