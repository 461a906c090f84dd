"""Split of a fused QKV accumulator: rescale, per-head norm, rotary embedding, store.

Drop-in for ``qkv_split`` and ``rope_inv_freq`` of ``instinctflash/kernels/rope.py`` (lines
22-114).  The raw accumulator of the fused projection holds ``[Q heads | K heads | V heads]``
per token; Q goes to ``q_out[t, h]``, K and V to row ``kv_base + t`` of their (cache) tensors,
``kv_base`` being an ``int`` or a one-element int32 device tensor that a captured graph re-reads.
Rotary angles are ``pos[t, sections[i]] * inv_freq[i]`` in float32 with split-half pairing.
"""
from __future__ import annotations

import torch

from .. import _lib
from ._common import launch, rows, vec

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def rope_inv_freq(head_dim, theta, device):
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64, device=device).float() / head_dim
    return (1.0 / (theta ** exponent)).float()


def _heads_out(t, name, n_heads, head_dim, dtype, device):
    if not isinstance(t, torch.Tensor) or t.ndim != 3:
        raise ValueError(f"{name} must be a 3-D tensor [rows, heads, head_dim]")
    if t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")
    if t.dtype != dtype:
        raise ValueError("q/k/v outputs must share a dtype")
    if t.shape[1] != n_heads or t.shape[2] != head_dim:
        raise ValueError(f"{name} must be [rows, {n_heads}, {head_dim}], got {tuple(t.shape)}")
    if head_dim > 1 and t.stride(2) != 1:
        raise ValueError(f"{name} must be contiguous in its last dimension")
    return t


def _index(t, name, n, device):
    if t is None:
        return None
    if t.dtype != torch.int32 or t.device != device or not t.is_contiguous() or t.numel() < n:
        raise ValueError(f"{name} must be a contiguous int32 tensor of at least {n} elements on {device}")
    return t


def qkv_split(qkv, q_out, k_out, v_out, *, heads_q, heads_kv, head_dim, row=None, col=None, bias=None,
              inv_freq=None, pos=None, sections=None, q_norm=None, k_norm=None, norm_eps=1e-6, kv_base=0):
    """q_out [T, HQ, HD]; k_out/v_out [S, HKV, HD] written at rows ``kv_base + t``."""
    if q_out.dtype != k_out.dtype or k_out.dtype != v_out.dtype:
        raise ValueError("q/k/v outputs must share a dtype")
    if q_out.dtype not in _FLOATS:
        raise ValueError(f"outputs have dtype {q_out.dtype}, expected one of {_FLOATS}")
    if inv_freq is not None and pos is None:
        raise ValueError("rotary needs a position table")
    if (q_norm is None) != (k_norm is None):
        raise ValueError("q_norm and k_norm come together")
    rows(qkv, "qkv", _FLOATS)
    T, width = qkv.shape
    n_heads = heads_q + 2 * heads_kv
    if head_dim % 2 or head_dim > 512:
        raise ValueError("head_dim must be even and at most 512")
    if width != n_heads * head_dim:
        raise ValueError(f"qkv must be [T, {n_heads * head_dim}], got {tuple(qkv.shape)}")
    dev = qkv.device
    _heads_out(q_out, "q_out", heads_q, head_dim, q_out.dtype, dev)
    _heads_out(k_out, "k_out", heads_kv, head_dim, q_out.dtype, dev)
    _heads_out(v_out, "v_out", heads_kv, head_dim, q_out.dtype, dev)
    if q_out.shape[0] < T:
        raise ValueError("q_out has fewer rows than qkv")
    half = head_dim // 2
    dynamic = torch.is_tensor(kv_base)
    if dynamic:
        _index(kv_base, "kv_base", 1, dev)
    else:
        if int(kv_base) < 0 or int(kv_base) + T > min(k_out.shape[0], v_out.shape[0]):
            raise ValueError("kv_base + T exceeds the rows of k_out / v_out")
    ld_pos = 0
    if pos is not None:
        if pos.dtype != torch.float32 or pos.ndim != 2 or pos.device != dev or pos.stride(1) != 1 and pos.shape[1] > 1:
            raise ValueError("pos must be a float32 [T, S] table on the same device")
        if pos.shape[0] < T:
            raise ValueError("pos has fewer rows than qkv")
        ld_pos = pos.stride(0)
    launch("iflb200_qkv_split", qkv,
        qkv.data_ptr(), _lib.dtype_code(qkv.dtype), qkv.stride(0) if T > 1 else width, T, int(heads_q), int(heads_kv),
        int(head_dim), _lib.ptr(vec(row, "row", T, dev)), _lib.ptr(vec(col, "col", width, dev)),
        _lib.ptr(vec(bias, "bias", width, dev)), _lib.ptr(vec(q_norm, "q_norm", head_dim, dev)),
        _lib.ptr(vec(k_norm, "k_norm", head_dim, dev)), float(norm_eps),
        _lib.ptr(vec(inv_freq, "inv_freq", half, dev)), _lib.ptr(pos), ld_pos,
        _lib.ptr(_index(sections, "sections", half, dev)), _lib.ptr(kv_base if dynamic else None),
        0 if dynamic else int(kv_base),
        q_out.data_ptr(), q_out.stride(0), q_out.stride(1), k_out.data_ptr(), k_out.stride(0), k_out.stride(1),
        v_out.data_ptr(), v_out.stride(0), v_out.stride(1), _lib.dtype_code(q_out.dtype))
