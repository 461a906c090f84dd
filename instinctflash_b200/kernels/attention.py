"""Merge of split-KV attention partials with the per-token FP8 quantiser of the merged row.

The reference's ``attention(..., split=workspace, q8=..., q8_scale=...)`` runs its attention
kernel over several key ranges and then ``_attn_combine`` (instinctflash/kernels/attention.py:109-145,
launched at :205-214), which merges the partial softmax states and can emit each token's full
output row as per-token e4m3 codes: the FP8 input of the O projection.  Attention itself is not
part of the FP8 linear path; this module provides the combine step with the same workspace layout
(``SplitWorkspace``, lines 148-158 there) and the same arithmetic, so the codes and scales are those
of the reference bit for bit.
"""
from __future__ import annotations

import torch

from .. import _lib
from ._common import E4M3, launch, ld, same_device


def _next_power_of_two(n: int) -> int:
    return 1 << max(0, (int(n) - 1).bit_length())


class SplitWorkspace:
    """Partial-softmax storage for split-KV attention of one fixed geometry (same fields and layout
    as the reference's class: ``po`` [splits, batch, hkv, rows, width], ``pm`` / ``pl``
    [splits, batch, hkv, rows], rows = tq * (hq // hkv), width = head_dim rounded up to a power of two)."""

    def __init__(self, batch, tq, hq, hkv, head_dim, splits, device):
        rows = tq * (hq // hkv)
        width = _next_power_of_two(head_dim)
        self.splits = splits
        self.po = torch.empty(splits * batch * hkv * rows * width, device=device, dtype=torch.float32)
        self.pm = torch.empty(splits * batch * hkv * rows, device=device, dtype=torch.float32)
        self.pl = torch.empty_like(self.pm)


def attn_combine(split: SplitWorkspace, out=None, *, heads_q: int, heads_kv: int, head_dim: int, tokens: int,
                 batch: int = 1, q8=None, q8_scale=None):
    """Merge the partials in ``split``; write ``out`` [B, Tq, Hq, D] (optional) and/or the quantised
    rows ``q8`` [Tq, Hq*D] e4m3 with ``q8_scale`` [Tq] (batch 1 only, as in the reference)."""
    if out is None and q8 is None:
        raise ValueError("nothing to write: give out, q8, or both")
    if heads_q % heads_kv:
        raise ValueError("heads_q must be a multiple of heads_kv")
    if head_dim % 4 or head_dim > 512 or heads_q * head_dim > 8192:
        raise ValueError("head_dim must be a multiple of 4, at most 512, and heads_q * head_dim at most 8192")
    for name in ("po", "pm", "pl"):
        t = getattr(split, name)
        if t.device.type != "cuda" or t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"split.{name} must be a contiguous float32 CUDA tensor; this path has no CPU implementation")
    rows = tokens * (heads_q // heads_kv)
    width = _next_power_of_two(head_dim)
    if split.pm.numel() < split.splits * batch * heads_kv * rows or split.po.numel() < split.splits * batch * heads_kv * rows * width:
        raise ValueError("the split workspace is smaller than the geometry asks for")
    if out is not None:
        if out.ndim != 4 or tuple(out.shape) != (batch, tokens, heads_q, head_dim) or out.stride(-1) != 1:
            raise ValueError("attention requires out [B, Tq, Hq, D] with a contiguous last dimension")
        if out.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise ValueError(f"unsupported output type {out.dtype}")
    if q8 is not None:
        if batch != 1:
            raise ValueError("fused FP8 output supports batch 1")
        if q8.dtype != E4M3 or q8.ndim != 2 or tuple(q8.shape) != (tokens, heads_q * head_dim) or q8.stride(1) != 1:
            raise ValueError(f"q8 must be e4m3 [{tokens}, {heads_q * head_dim}] with a contiguous last dimension")
        if q8_scale is None or q8_scale.dtype != torch.float32 or q8_scale.numel() < tokens or not q8_scale.is_contiguous():
            raise ValueError("q8_scale must be a contiguous float32 vector with one entry per token")
    same_device(split.po, pm=split.pm, pl=split.pl, out=out, q8=q8, q8_scale=q8_scale)
    launch("iflb200_attn_combine_quant", split.po, split.po.data_ptr(), split.pm.data_ptr(), split.pl.data_ptr(),
           int(split.splits), int(batch), int(tokens), int(heads_q), int(heads_kv), int(head_dim),
           _lib.ptr(out), _lib.dtype_code(out.dtype) if out is not None else _lib.F32,
           out.stride(0) if out is not None else 0, out.stride(1) if out is not None else 0,
           out.stride(2) if out is not None else 0,
           _lib.ptr(q8), ld(q8) if q8 is not None else 0, _lib.ptr(q8_scale))
    return out
