"""bf16 -> e4m3 packing with a fixed or a dynamic per-tensor scale.

Drop-in for ``instinctflash/runtime/fp8_pack.py``: ``pack_bf16_e4m3(x, scale)`` (lines 44-60)
and ``dynamic_pack_bf16_e4m3(x) -> (packed, scale)`` (lines 83-92) with the same arithmetic:
amax with NaN propagation, ``scale = max(amax, 1e-12) * fp32(1/448)``, IEEE division,
NaN-propagating clamp to +-448 and a round-to-nearest-even cast.  Two launches instead of the
reference's three; like the reference, the dynamic form allocates its output, its scale and
a small partial-maximum buffer per call.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..kernels._common import launch


def _check(x):
    if x.device.type != "cuda":
        raise ValueError("FP8 packing requires a CUDA tensor; this path has no CPU implementation")
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("FP8 packing requires contiguous BF16 inputs")


def pack_bf16_e4m3(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    _check(x)
    if scale.dtype != torch.float32 or scale.numel() != 1 or scale.device != x.device:
        raise ValueError("FP8 packing requires one FP32 scale on the input device")
    out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    if x.numel():
        launch("iflb200_pack_bf16_e4m3", x, x.data_ptr(), x.numel(), scale.data_ptr(), out.data_ptr())
    return out


def dynamic_pack_bf16_e4m3(x: torch.Tensor):
    _check(x)
    if not x.numel():
        raise ValueError("Dynamic FP8 packing requires nonempty contiguous CUDA BF16 input")
    lib = _lib.lib()
    n = x.numel()
    nbytes = int(lib.iflb200_pack_workspace_bytes(n))
    workspace = torch.empty((nbytes + 3) // 4, device=x.device, dtype=torch.int32)
    scale = torch.empty((1,), device=x.device, dtype=torch.float32)
    out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    launch("iflb200_dynamic_pack_bf16_e4m3", x, x.data_ptr(), n, out.data_ptr(), scale.data_ptr(),
           workspace.data_ptr(), nbytes)
    return out, scale
