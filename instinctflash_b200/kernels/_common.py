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


class on_device:
    """Make ``t``'s device the current CUDA device around a call into the library.

    The library keys everything on the current device (SM count, kernel attributes, the launch
    itself), so a call made while another GPU is current would launch there with this GPU's
    pointers.  The device is switched only when it differs, and restored afterwards."""

    def __init__(self, t: torch.Tensor):
        self.index = t.device.index if t.device.index is not None else torch.cuda.current_device()
        self.previous = None

    def __enter__(self):
        current = torch.cuda.current_device()
        if current != self.index:
            self.previous = current
            torch.cuda.set_device(self.index)
        return self

    def __exit__(self, *exc):
        if self.previous is not None:
            torch.cuda.set_device(self.previous)
        return False


def launch(entry: str, anchor: torch.Tensor, *args) -> None:
    """Call ``entry`` of the library on ``anchor``'s device and current stream (the stream handle
    is every entry point's last argument); raise on a non-zero status.  Tensor arguments on
    another device than ``anchor`` are refused before anything is launched."""
    with on_device(anchor):
        status = getattr(_lib.lib(), entry)(*args, _lib.stream_handle(anchor.device))
    _lib.check(status, entry.removeprefix("iflb200_"))


def same_device(anchor: torch.Tensor, **tensors) -> None:
    for name, t in tensors.items():
        if t is not None and t.device != anchor.device:
            raise ValueError(f"{name} is on {t.device}, expected {anchor.device}")
