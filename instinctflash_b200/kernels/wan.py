"""Wan-DiT projection consumer: full-width Q/K RMS norm, interleaved rotary, pooled K/V.

Drop-in for ``wan_qkv`` of ``instinctflash/kernels/wan.py`` (lines 20-104).  One token row of
a raw fused accumulator ``[Q | K | V]`` (each ``heads * head_dim`` wide; K and V only when
their pools are given) is dequantised, Q and K are RMS-normalised over their full width,
adjacent channel pairs ``(2j, 2j+1)`` of every head are rotated by
``pos[t, sections[j]] * inv_freq[j]``, Q is stored densely and K/V go to pool rows
``slots[t]`` of batch ``row // tokens``.
"""
from __future__ import annotations

import torch

from .. import _lib
from ._common import launch, rows, vec
from .rope import _FLOATS, _index


def _pool(t, name, D, dtype, device):
    if t is None:
        return None
    if t.ndim != 3 or t.shape[2] != D or (D > 1 and t.stride(2) != 1):
        raise ValueError(f"{name} must be [B, S, {D}] and contiguous in its last dimension")
    if t.dtype != dtype or t.device != device:
        raise ValueError(f"{name} must share q_out's dtype and device")
    return t


def wan_qkv(raw, q_out, *, heads, head_dim, tokens, k_pool=None, v_pool=None, slots=None, row=None, col=None,
            bias=None, q_norm=None, k_norm=None, pos=None, sections=None, inv_freq=None, eps=1e-6, num_warps=8):
    """raw [B*T, parts*H*HD] (parts: Q, then K, then V); q_out [B*T, H*HD];
    k_pool / v_pool [B, S, H*HD] written at rows ``slots[t]`` (or ``t``)."""
    rows(raw, "raw", _FLOATS)
    rows(q_out, "q_out", _FLOATS)
    n_rows = raw.shape[0]
    D = heads * head_dim
    if head_dim % 2 or head_dim > 512 or D > 8192:
        raise ValueError("head_dim must be even and at most 512, heads * head_dim at most 8192")
    if v_pool is not None and k_pool is None:
        raise ValueError("parts are Q, then K, then V: a V pool needs a K pool")
    parts = 1 + (k_pool is not None) + (v_pool is not None)
    if raw.shape[1] < parts * D:
        raise ValueError(f"raw must be at least [rows, {parts * D}], got {tuple(raw.shape)}")
    if tuple(q_out.shape) != (n_rows, D):
        raise ValueError(f"q_out must be [{n_rows}, {D}], got {tuple(q_out.shape)}")
    if tokens <= 0 or n_rows % tokens:
        raise ValueError("rows must be a whole number of batches of `tokens` rows")
    dev = raw.device
    _pool(k_pool, "k_pool", D, q_out.dtype, dev)
    _pool(v_pool, "v_pool", D, q_out.dtype, dev)
    half = head_dim // 2
    if inv_freq is not None and (pos is None or sections is None):
        raise ValueError("rotary needs a position table and the section map")
    ld_pos = 0
    if pos is not None:
        if pos.dtype != torch.float32 or pos.ndim != 2 or pos.device != dev or (pos.shape[1] > 1 and pos.stride(1) != 1):
            raise ValueError("pos must be a float32 [T, S] table on the same device")
        if pos.shape[0] < tokens:
            raise ValueError("pos has fewer rows than tokens")
        ld_pos = pos.stride(0)
    kp, vp = k_pool, v_pool
    launch("iflb200_wan_qkv", raw,
        raw.data_ptr(), _lib.dtype_code(raw.dtype), raw.stride(0) if n_rows > 1 else raw.shape[1], n_rows, int(tokens),
        int(heads), int(head_dim), _lib.ptr(vec(row, "row", n_rows, dev)), _lib.ptr(vec(col, "col", parts * D, dev)),
        _lib.ptr(vec(bias, "bias", parts * D, dev)), _lib.ptr(vec(q_norm, "q_norm", D, dev)),
        _lib.ptr(vec(k_norm, "k_norm", D, dev)), float(eps), _lib.ptr(vec(inv_freq, "inv_freq", half, dev)),
        _lib.ptr(pos), ld_pos, _lib.ptr(_index(sections, "sections", half, dev)),
        _lib.ptr(_index(slots, "slots", tokens, dev)),
        q_out.data_ptr(), q_out.stride(0) if n_rows > 1 else D,
        _lib.ptr(kp), kp.stride(0) if kp is not None else 0, kp.stride(1) if kp is not None else 0,
        _lib.ptr(vp), vp.stride(0) if vp is not None else 0, vp.stride(1) if vp is not None else 0,
        _lib.dtype_code(q_out.dtype))
