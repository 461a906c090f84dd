"""Argument checks shared by the operator wrappers (raise before anything is launched)."""
from __future__ import annotations

import torch

from .. import _lib

E4M3 = torch.float8_e4m3fn


def rows(t: torch.Tensor, name: str, dtypes=None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.ndim != 2:
        raise ValueError(f"{name} must be 2-D [rows, width], got shape {tuple(t.shape)}")
    if t.device.type != "cuda":
        raise ValueError(f"{name} must live on a CUDA device; this path has no CPU implementation")
    if t.shape[1] > 1 and t.stride(1) != 1:
        raise ValueError(f"{name} must be contiguous in its last dimension")
    if dtypes is not None and t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {tuple(dtypes)}")
    return t


def vec(t, name: str, n: int, device) -> torch.Tensor | None:
    """Optional float32 vector of ``n`` elements (or a flat table) on ``device``."""
    if t is None:
        return None
    if t.dtype != torch.float32:
        raise ValueError(f"{name} must be float32, got {t.dtype}")
    if t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if n is not None and t.numel() < n:
        raise ValueError(f"{name} has {t.numel()} elements, expected at least {n}")
    return t


def ld(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def stream(t: torch.Tensor) -> int:
    return _lib.stream_handle(t.device)
