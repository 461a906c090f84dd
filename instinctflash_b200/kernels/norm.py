"""Row producers and consumers around the FP8 GEMM.

Drop-in for the three operators of ``instinctflash/kernels/norm.py``:
``row_quant`` (lines 128-158), ``dequant_rows`` (lines 162-185) and ``residual_norm_quant``
(lines 26-124, without its MoE ``router`` tail).  Same argument names and meaning; the Triton
tuning hints (``num_warps``, ``block``) are accepted and ignored.  The arithmetic follows the
instruction order the reference compiles to on sm_100, so the e4m3 codes and scales of the
quantiser are bit-identical to the reference's on the same inputs.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ._common import E4M3, launch, ld, rows, same_device, vec

FP8_MAX = 448.0
_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def row_quant(x, q, q_scale, *, row=None, col=None, bias=None, gelu=False, num_warps=None):
    """q[m] = e4m3((x[m] * row[m] * col + bias) [-> gelu_tanh] / s[m]), s[m] = rowmax / 448."""
    rows(x, "x", _FLOATS)
    rows(q, "q", (E4M3,))
    M, D = x.shape
    if tuple(q.shape) != (M, D):
        raise ValueError(f"q must be [{M}, {D}], got {tuple(q.shape)}")
    vec(q_scale, "q_scale", M, x.device)
    same_device(x, q=q)
    launch("iflb200_row_quant", x,
        x.data_ptr(), _lib.dtype_code(x.dtype), ld(x), M, D,
        _lib.ptr(vec(row, "row", M, x.device)), _lib.ptr(vec(col, "col", D, x.device)),
        _lib.ptr(vec(bias, "bias", D, x.device)), int(bool(gelu)),
        q.data_ptr(), ld(q), q_scale.data_ptr())


def row_quant_sharded(x, q, q_scale, amax, phase, *, row=None, col=None, bias=None, gelu=False):
    """The quantiser for rows whose columns are sharded over GPUs (no reference counterpart:
    the reference is single-GPU).  ``phase=1`` writes the local row maxima to ``amax`` [M];
    after an all-reduce-max of ``amax`` over the shards, ``phase=2`` writes ``q`` and ``q_scale``
    from the global maxima: bit-identical to the codes of the unsharded row."""
    rows(x, "x", _FLOATS)
    M, D = x.shape
    vec(amax, "amax", M, x.device)
    if phase in (2, 3):
        rows(q, "q", (E4M3,))
        if tuple(q.shape) != (M, D):
            raise ValueError(f"q must be [{M}, {D}], got {tuple(q.shape)}")
        vec(q_scale, "q_scale", M, x.device)
    elif phase != 1:
        raise ValueError("phase must be 1 (local maxima), 2 (quantise with the reduced maxima) or 3 (2, then zero them)")
    same_device(x, q=q if phase != 1 else None)
    launch("iflb200_row_quant_sharded", x,
        x.data_ptr(), _lib.dtype_code(x.dtype), ld(x), M, D,
        _lib.ptr(vec(row, "row", M, x.device)), _lib.ptr(vec(col, "col", D, x.device)),
        _lib.ptr(vec(bias, "bias", D, x.device)), int(bool(gelu)), int(phase), amax.data_ptr(),
        _lib.ptr(q) if phase != 1 else None, ld(q) if phase != 1 else 0,
        _lib.ptr(q_scale) if phase != 1 else None)


def row_max_sharded(x, amax, mirrors=(), *, row=None, col=None, bias=None, gelu=False):
    """Phase 1 of ``row_quant_sharded`` that also writes the row maxima into ``mirrors`` (up to 7
    float32 [M] buffers: this rank's slots in the other GPUs' peer-mapped buffers)."""
    rows(x, "x", _FLOATS)
    M, D = x.shape
    vec(amax, "amax", M, x.device)
    if len(mirrors) > 7:
        raise ValueError("at most 7 mirrors")
    for t in mirrors:
        vec(t, "amax mirror", M, x.device)
    n = len(mirrors)
    launch("iflb200_row_max_sharded", x, x.data_ptr(), _lib.dtype_code(x.dtype), ld(x), M, D,
           _lib.ptr(vec(row, "row", M, x.device)), _lib.ptr(vec(col, "col", D, x.device)),
           _lib.ptr(vec(bias, "bias", D, x.device)), int(bool(gelu)), amax.data_ptr(),
           (ctypes.c_void_p * n)(*[t.data_ptr() for t in mirrors]) if n else None, n)


def row_quant_from_amax(h, amax, q, q_scale):
    """Second half of ``fp8.fp8_linear_gated``: quantise the rows of ``h`` [M, F] float32 with the
    row maxima the GEMM epilogue left in ``amax`` [M] (scale = amax / 448, codes as ``row_quant``),
    and leave ``amax`` at zero for the next call."""
    row_quant_sharded(h, q, q_scale, amax, 3)


def quant_from_amax(h, amax, q, q_scale, zero=None):
    """``row_quant_from_amax`` as a flat kernel (rows cut into pieces for separate CTAs): the same
    codes and scales; ``amax`` is left as it is and ``zero`` (another [M] float32 buffer, or None) is
    cleared instead -- two buffers of row maxima alternate between consecutive gated GEMMs."""
    rows(h, "h", (torch.float32,))
    M, F = h.shape
    rows(q, "q", (E4M3,))
    if tuple(q.shape) != (M, F):
        raise ValueError(f"q must be [{M}, {F}], got {tuple(q.shape)}")
    vec(amax, "amax", M, h.device)
    vec(q_scale, "q_scale", M, h.device)
    if zero is not None:
        vec(zero, "zero", M, h.device)
        if zero.data_ptr() == amax.data_ptr():
            raise ValueError("zero must be another buffer than amax")
    same_device(h, q=q)
    launch("iflb200_quant_from_amax", h, h.data_ptr(), ld(h), M, F, amax.data_ptr(), _lib.ptr(zero), q.data_ptr(), ld(q),
           q_scale.data_ptr())


def dequant_rows(x, y, *, row=None, col=None, bias=None, block=None, num_warps=4):
    """y[m] = x[m] * row[m] * col + bias (float dtypes in and out)."""
    rows(x, "x", _FLOATS)
    rows(y, "y", _FLOATS)
    M, D = x.shape
    if tuple(y.shape) != (M, D):
        raise ValueError(f"y must be [{M}, {D}], got {tuple(y.shape)}")
    same_device(x, y=y)
    launch("iflb200_dequant_rows", x,
        x.data_ptr(), _lib.dtype_code(x.dtype), ld(x), M, D,
        _lib.ptr(vec(row, "row", M, x.device)), _lib.ptr(vec(col, "col", D, x.device)),
        _lib.ptr(vec(bias, "bias", D, x.device)),
        y.data_ptr(), _lib.dtype_code(y.dtype), ld(y))


def residual_norm_quant(res, *, delta=None, delta_row=None, delta_col=None, bias=None, gate=None,
                        write_res=True, layernorm=False, weight=None, beta=None,
                        mod_scale=None, mod_shift=None, q=None, q_scale=None, y=None, eps=1e-6,
                        num_warps=None, router=None, mod_index=None):
    """Residual update, RMS/LayerNorm, affine, adaptive modulation and per-token quantiser.

        if delta:  res[m] += (delta[m] * delta_row[m] * delta_col + bias) * gate
        y[m] = norm(res[m]) * weight + beta;  y[m] = y[m] * (1 + mod_scale) + mod_shift
        q[m], s[m] = e4m3(y[m] / s[m]), rowmax(|y[m]|) / 448

    ``res`` is float32 (bf16 for the Wan residual stream) and updated in place; ``gate``,
    ``mod_scale`` and ``mod_shift`` are [D] or, with ``mod_index`` (int32 [M]), tables [n, D].
    """
    return _residual_norm_quant(res, delta, delta_row, delta_col, bias, gate, write_res, layernorm, weight, beta,
                                mod_scale, mod_shift, q, q_scale, y, eps, router, mod_index, None, None)


def residual_norm_quant_peers(res, *, delta, q, q_scale, q_mirrors, q_scale_mirrors, delta_row=None, delta_col=None,
                              bias=None, gate=None, write_res=True, layernorm=False, weight=None, beta=None,
                              mod_scale=None, mod_shift=None, eps=1e-6, mod_index=None):
    """``residual_norm_quant`` for the row owner of a tensor-parallel group: ``delta`` [p, M, D]
    float32 holds the ranks' partial sums of these rows (added in rank order, then rounded to bf16);
    the codes and row scales also go into ``q_mirrors`` / ``q_scale_mirrors`` (up to 7 each): the
    same rows of the other GPUs' replicas of the next block's input, peer-mapped."""
    return _residual_norm_quant(res, delta, delta_row, delta_col, bias, gate, write_res, layernorm, weight, beta,
                                mod_scale, mod_shift, q, q_scale, None, eps, None, mod_index, list(q_mirrors),
                                list(q_scale_mirrors))


def _residual_norm_quant(res, delta, delta_row, delta_col, bias, gate, write_res, layernorm, weight, beta, mod_scale,
                         mod_shift, q, q_scale, y, eps, router, mod_index, q_mirrors, q_scale_mirrors):
    if router is not None:
        raise NotImplementedError("the MoE router tail of residual_norm_quant is outside the FP8 linear path")
    rows(res, "res", (torch.float32, torch.bfloat16))
    M, D = res.shape
    dev = res.device
    partials = delta is not None and delta.ndim == 3
    if partials:
        # fp32 partial sums of a K-split GEMM (fp8.gemm_partials): [S, M, D], added in split order
        if delta.dtype != torch.float32 or tuple(delta.shape[1:]) != (M, D) or not delta.is_contiguous() or not 1 <= delta.shape[0] <= 8:
            raise ValueError(f"split-K partial sums must be a contiguous float32 [S <= 8, {M}, {D}] tensor")
        if delta.device.type != "cuda":
            raise ValueError("delta must live on a CUDA device; this path has no CPU implementation")
    elif delta is not None:
        rows(delta, "delta", (torch.bfloat16,))
        if tuple(delta.shape) != (M, D):
            raise ValueError(f"delta must be [{M}, {D}], got {tuple(delta.shape)}")
    if q is not None:
        rows(q, "q", (E4M3,))
        if tuple(q.shape) != (M, D):
            raise ValueError(f"q must be [{M}, {D}], got {tuple(q.shape)}")
        if q_scale is None:
            raise ValueError("q_scale is required with q")
        vec(q_scale, "q_scale", M, dev)
    if y is not None:
        rows(y, "y", _FLOATS)
        if tuple(y.shape) != (M, D):
            raise ValueError(f"y must be [{M}, {D}], got {tuple(y.shape)}")
    if (mod_scale is None) != (mod_shift is None):
        raise ValueError("mod_scale and mod_shift come together")
    if mod_index is not None and (mod_index.dtype != torch.int32 or mod_index.numel() < M):
        raise ValueError("mod_index must be int32 with one entry per row")
    same_device(res, delta=delta, q=q, y=y, mod_index=mod_index)
    if q_mirrors:
        if not partials or q is None or y is not None or len(q_mirrors) != len(q_scale_mirrors or ()) or len(q_mirrors) > 7:
            raise ValueError("mirrors go with the partial-sum form: q without y, as many scale mirrors as code mirrors, at most 7")
        for t in q_mirrors:
            rows(t, "q mirror", (E4M3,))
            if tuple(t.shape) != (M, D) or ld(t) != ld(q):
                raise ValueError("a q mirror must have q's shape and row stride")
        for t in q_scale_mirrors:
            vec(t, "q_scale mirror", M, dev)
        n = len(q_mirrors)
        launch("iflb200_residual_norm_quant_peers", res,
            res.data_ptr(), _lib.dtype_code(res.dtype), ld(res), M, D, delta.data_ptr(), int(delta.shape[0]), D,
            _lib.ptr(vec(delta_row, "delta_row", M, dev)), _lib.ptr(vec(delta_col, "delta_col", D, dev)),
            _lib.ptr(vec(bias, "bias", D, dev)), _lib.ptr(vec(gate, "gate", D, dev)), int(bool(write_res)),
            int(bool(layernorm)), _lib.ptr(vec(weight, "weight", D, dev)), _lib.ptr(vec(beta, "beta", D, dev)),
            _lib.ptr(vec(mod_scale, "mod_scale", D, dev)), _lib.ptr(vec(mod_shift, "mod_shift", D, dev)),
            _lib.ptr(mod_index), float(eps), _lib.ptr(q), ld(q), _lib.ptr(q_scale),
            (ctypes.c_void_p * n)(*[t.data_ptr() for t in q_mirrors]),
            (ctypes.c_void_p * n)(*[t.data_ptr() for t in q_scale_mirrors]), n)
        return
    launch("iflb200_residual_norm_quant_partials" if partials else "iflb200_residual_norm_quant", res,
        res.data_ptr(), _lib.dtype_code(res.dtype), ld(res), M, D,
        *((delta.data_ptr(), int(delta.shape[0]), D) if partials else
          (_lib.ptr(delta), ld(delta) if delta is not None else 0)),
        _lib.ptr(vec(delta_row, "delta_row", M, dev)), _lib.ptr(vec(delta_col, "delta_col", D, dev)),
        _lib.ptr(vec(bias, "bias", D, dev)), _lib.ptr(vec(gate, "gate", D, dev)), int(bool(write_res)),
        int(bool(layernorm)), _lib.ptr(vec(weight, "weight", D, dev)), _lib.ptr(vec(beta, "beta", D, dev)),
        _lib.ptr(vec(mod_scale, "mod_scale", D, dev)), _lib.ptr(vec(mod_shift, "mod_shift", D, dev)),
        _lib.ptr(mod_index), float(eps),
        _lib.ptr(q), ld(q) if q is not None else 0, _lib.ptr(q_scale),
        _lib.ptr(y), _lib.dtype_code(y.dtype) if y is not None else _lib.F32,
        ld(y) if y is not None else 0)
