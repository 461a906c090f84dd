"""numpy/torch front end of the C restatement (``fp8_linear_oracle.c``).

All inputs and outputs are CPU torch tensors.  Each function names the reference operator it
restates; the arithmetic itself is in the C file (exact ``fmaf``, explicit rounding).
TEST INFRASTRUCTURE ONLY — see the package docstring.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import build as _build

E4M3 = torch.float8_e4m3fn
F32, BF16, F16 = 0, 1, 2
_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(_build.build()))
        _LIB.oracle_e4m3_encode.restype = ctypes.c_uint8
        _LIB.oracle_e4m3_encode.argtypes = [ctypes.c_float]
        _LIB.oracle_e4m3_decode.restype = ctypes.c_float
        _LIB.oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
    return _LIB


def _f32(t):
    """Contiguous float32 numpy copy of a float tensor (widening is exact)."""
    return None if t is None else np.ascontiguousarray(t.detach().to(torch.float32).cpu().numpy())


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _codes(t):
    return np.ascontiguousarray(t.detach().cpu().contiguous().view(torch.uint8).numpy())


def _as_e4m3(codes: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(codes).view(E4M3)


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 codes by the integer round-to-nearest-even cast
    (instinctflash/runtime/fp8_pack.py:12-23; same result as cvt.rn.satfinite)."""
    flat = x.detach().to(torch.float32).flatten().tolist()
    lib = _lib()
    out = np.fromiter((lib.oracle_e4m3_encode(v) for v in flat), dtype=np.uint8, count=len(flat))
    return _as_e4m3(out.reshape(tuple(x.shape)))


def quantize_weight(w: torch.Tensor, bias=None, *, reciprocal: bool = False):
    """Per-output-channel pack (instinctflash/kernels/fp8.py:30-37).

    ``reciprocal=False`` is torch's CPU arithmetic (true division by 448); ``True`` is its CUDA
    arithmetic for tensor / python-scalar (multiply by fp32(1/448)), as the reference documents
    at instinctflash/runtime/torch_fp8_linear.py:41-46.  Returns (codes e4m3 [N,K], scale, bias).
    """
    wf = w.detach().to(torch.float32).cpu()
    amax = wf.abs().amax(dim=1).clamp_min(1e-12)
    scale = amax * torch.tensor(1.0 / 448.0, dtype=torch.float32) if reciprocal else amax / 448.0
    q = (wf / scale[:, None]).clamp_(-448.0, 448.0).to(E4M3)
    b = None if bias is None else bias.detach().to(torch.float32).cpu().contiguous()
    return q.contiguous(), scale.contiguous(), b


def row_quant(x, *, row=None, col=None, bias=None, gelu=False):
    """instinctflash/kernels/norm.py:128-147 -> (codes e4m3 [M,K], scales f32 [M])."""
    xf = _f32(x)
    M, K = xf.shape
    q = np.empty((M, K), np.uint8)
    qs = np.empty((M,), np.float32)
    r, c, b = _f32(row), _f32(col), _f32(bias)
    _lib().oracle_row_quant(_p(xf), ctypes.c_int64(K), M, K, _p(r), _p(c), _p(b), int(gelu), _p(q),
                            ctypes.c_int64(K), _p(qs))
    return _as_e4m3(q), torch.from_numpy(qs)


def row_quant_sharded(x, amax, phase, *, row=None, col=None, bias=None, gelu=False):
    """Two-phase quantiser for column-sharded rows (the tensor-parallel split of
    instinctflash/kernels/norm.py:128-147).  phase 1 -> local row maxima [M];
    phase 2 (amax = reduced maxima) -> (codes, scales)."""
    xf = _f32(x)
    M, K = xf.shape
    r, c, b = _f32(row), _f32(col), _f32(bias)
    am = np.ascontiguousarray(amax.detach().cpu().numpy().astype(np.float32)) if phase == 2 else np.empty((M,), np.float32)
    q = np.empty((M, K), np.uint8)
    qs = np.empty((M,), np.float32)
    _lib().oracle_row_quant_sharded(_p(xf), ctypes.c_int64(K), M, K, _p(r), _p(c), _p(b), int(gelu), int(phase),
                                    _p(am), _p(q), ctypes.c_int64(K), _p(qs))
    if phase == 1:
        return torch.from_numpy(am)
    return _as_e4m3(q), torch.from_numpy(qs)


def dequant_rows(x, *, row=None, col=None, bias=None, out_dtype=torch.bfloat16):
    """instinctflash/kernels/norm.py:162-175 -> y [M,D] in out_dtype."""
    xf = _f32(x)
    M, D = xf.shape
    y = np.empty((M, D), np.float32)
    r, c, b = _f32(row), _f32(col), _f32(bias)
    _lib().oracle_dequant_rows(_p(xf), ctypes.c_int64(D), M, D, _p(r), _p(c), _p(b), _p(y), ctypes.c_int64(D),
                               _DT[out_dtype])
    return torch.from_numpy(y).to(out_dtype)


def gated_act_quant(gu, *, row=None, col=None, act=0):
    """instinctflash/kernels/activation.py:20-43 -> (codes [M,F], scales [M])."""
    gf = _f32(gu)
    M, F2 = gf.shape
    F = F2 // 2
    q = np.empty((M, F), np.uint8)
    qs = np.empty((M,), np.float32)
    r, c = _f32(row), _f32(col)
    _lib().oracle_gated_act_quant(_p(gf), ctypes.c_int64(F2), M, F, _p(r), _p(c), int(act), _p(q),
                                  ctypes.c_int64(F), _p(qs))
    return _as_e4m3(q), torch.from_numpy(qs)


def residual_norm_quant(res, *, delta=None, delta_row=None, delta_col=None, bias=None, gate=None,
                        write_res=True, layernorm=False, weight=None, beta=None, mod_scale=None,
                        mod_shift=None, mod_index=None, eps=1e-6, quant=True, y_dtype=None):
    """instinctflash/kernels/norm.py:26-94 (no router).

    Returns dict(res=updated residual in res.dtype, q=codes|None, qs=scales|None, y=tensor|None).
    """
    rf = _f32(res)
    M, D = rf.shape
    d = _f32(delta)
    q = np.empty((M, D), np.uint8) if quant else None
    qs = np.empty((M,), np.float32) if quant else None
    y = np.empty((M, D), np.float32) if y_dtype is not None else None
    args = [_f32(t) for t in (delta_row, delta_col, bias, gate)]
    w, b, ms, mh = _f32(weight), _f32(beta), _f32(mod_scale), _f32(mod_shift)
    mi = None if mod_index is None else np.ascontiguousarray(mod_index.cpu().numpy().astype(np.int32))
    _lib().oracle_residual_norm_quant(
        _p(rf), ctypes.c_int64(D), _DT[res.dtype], M, D, _p(d), ctypes.c_int64(D), *[_p(a) for a in args],
        int(bool(write_res)), int(bool(layernorm)), _p(w), _p(b), _p(ms), _p(mh), _p(mi), ctypes.c_float(eps),
        _p(q), ctypes.c_int64(D), _p(qs), _p(y), ctypes.c_int64(D), _DT[y_dtype] if y_dtype is not None else 0)
    return dict(res=torch.from_numpy(rf).to(res.dtype),
                q=None if q is None else _as_e4m3(q),
                qs=None if qs is None else torch.from_numpy(qs),
                y=None if y is None else torch.from_numpy(y).to(y_dtype))


def _i32(t):
    return None if t is None else np.ascontiguousarray(t.detach().cpu().numpy().astype(np.int32))


def qkv_split(qkv, *, heads_q, heads_kv, head_dim, kv_rows, row=None, col=None, bias=None, inv_freq=None,
              pos=None, sections=None, q_norm=None, k_norm=None, norm_eps=1e-6, kv_base=0,
              out_dtype=torch.float16):
    """instinctflash/kernels/rope.py:22-83 -> (q [T,HQ,HD], k [kv_rows,HKV,HD], v likewise), rows
    outside ``kv_base .. kv_base+T`` of k and v left at zero."""
    xf = _f32(qkv)
    T = xf.shape[0]
    q = np.zeros((T, heads_q, head_dim), np.float32)
    k = np.zeros((kv_rows, heads_kv, head_dim), np.float32)
    v = np.zeros_like(k)
    pf = _f32(pos)
    _lib().oracle_qkv_split(_p(xf), ctypes.c_int64(xf.shape[1]), T, heads_q, heads_kv, head_dim, _p(_f32(row)),
                            _p(_f32(col)), _p(_f32(bias)), _p(_f32(q_norm)), _p(_f32(k_norm)),
                            ctypes.c_float(norm_eps), _p(_f32(inv_freq)), _p(pf),
                            ctypes.c_int64(0 if pf is None else pf.shape[1]), _p(_i32(sections)), int(kv_base),
                            _p(q), _p(k), _p(v), _DT[out_dtype])
    return tuple(torch.from_numpy(a).to(out_dtype) for a in (q, k, v))


def wan_qkv(raw, *, heads, head_dim, tokens, parts, pool_rows=None, slots=None, row=None, col=None, bias=None,
            q_norm=None, k_norm=None, pos=None, sections=None, inv_freq=None, eps=1e-6,
            out_dtype=torch.bfloat16):
    """instinctflash/kernels/wan.py:20-82 -> (q [rows,D], k_pool [B,S,D] or None, v_pool or None)."""
    xf = _f32(raw)
    n_rows = xf.shape[0]
    D = heads * head_dim
    B = n_rows // tokens
    S = pool_rows if pool_rows is not None else tokens
    q = np.zeros((n_rows, D), np.float32)
    kp = np.zeros((B, S, D), np.float32) if parts >= 2 else None
    vp = np.zeros((B, S, D), np.float32) if parts >= 3 else None
    pf = _f32(pos)
    _lib().oracle_wan_qkv(_p(xf), ctypes.c_int64(xf.shape[1]), n_rows, tokens, heads, head_dim, parts,
                          _p(_f32(row)), _p(_f32(col)), _p(_f32(bias)), _p(_f32(q_norm)), _p(_f32(k_norm)),
                          ctypes.c_float(eps), _p(_f32(inv_freq)), _p(pf),
                          ctypes.c_int64(0 if pf is None else pf.shape[1]), _p(_i32(sections)), _p(_i32(slots)),
                          S, _p(q), _p(kp), _p(vp), _DT[out_dtype])
    return tuple(None if a is None else torch.from_numpy(a).to(out_dtype) for a in (q, kp, vp))


def gemm_acc(a, w):
    """fp32_rn of the exact sum_k a[m,k]*w[n,k] over e4m3 codes -> float32 [M,N]."""
    ac, wc = _codes(a), _codes(w)
    M, K = ac.shape
    N = wc.shape[0]
    out = np.empty((M, N), np.float32)
    _lib().oracle_gemm_acc(_p(ac), ctypes.c_int64(K), _p(wc), ctypes.c_int64(K), M, N, K, _p(out), ctypes.c_int64(N))
    return torch.from_numpy(out)


def gemm(a, w):
    """instinctflash/kernels/fp8.py:50-53: raw accumulator rounded to bf16."""
    return gemm_acc(a, w).to(torch.bfloat16)


def fp8_linear(a, a_scale, w, w_scale, bias=None, *, exact=False, out_dtype=torch.bfloat16):
    """gemm (fp8.py:50-53) + dequant_rows (norm.py:162-175); ``exact`` skips the bf16 rounding of
    the accumulator (the single-rounding form that the dequantise-and-matmul baseline and
    torch._scaled_mm-with-scales approximate, torch_fp8_linear.py:74-78)."""
    ac, wc = _codes(a), _codes(w)
    M, K = ac.shape
    N = wc.shape[0]
    y = np.empty((M, N), np.float32)
    r, c, b = _f32(a_scale), _f32(w_scale), _f32(bias)
    rstride = 0 if (r is not None and r.size == 1 and M != 1) else 1
    cstride = 0 if (c is not None and c.size == 1 and N != 1) else 1
    _lib().oracle_fp8_linear(_p(ac), ctypes.c_int64(K), _p(wc), ctypes.c_int64(K), M, N, K, _p(r), rstride, _p(c),
                             cstride, _p(b), int(bool(exact)), _p(y), ctypes.c_int64(N), _DT[out_dtype])
    return torch.from_numpy(y).to(out_dtype)


def dynamic_pack_bf16_e4m3(x: torch.Tensor):
    """instinctflash/runtime/fp8_pack.py:62-92 -> (codes like x, scale f32 [1])."""
    bits = np.ascontiguousarray(x.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16))
    q = np.empty(bits.shape, np.uint8)
    scale = np.zeros((1,), np.float32)
    _lib().oracle_pack_tensor(_p(bits), ctypes.c_int64(bits.size), 1, _p(scale), _p(q))
    return _as_e4m3(q), torch.from_numpy(scale)


def pack_bf16_e4m3(x: torch.Tensor, scale: torch.Tensor):
    """instinctflash/runtime/fp8_pack.py:27-60 with a given scale."""
    bits = np.ascontiguousarray(x.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16))
    q = np.empty(bits.shape, np.uint8)
    s = np.ascontiguousarray(scale.detach().cpu().numpy().astype(np.float32).reshape(1))
    _lib().oracle_pack_tensor(_p(bits), ctypes.c_int64(bits.size), 0, _p(s), _p(q))
    return _as_e4m3(q)


def decode(q: torch.Tensor) -> torch.Tensor:
    return q.to(torch.float32)


def dequantise_and_matmul(q, s_x, wq, s_w, bias=None, out_dtype=torch.bfloat16):
    """The reference's CPU-runnable torch form of the linear
    (benchmarks/native/fp8_probe.py:32-36): ((q*s_x) @ (Wq*s_w)^T + b) in fp32, then out_dtype."""
    y = (q.to(torch.float32) * s_x[:, None]) @ (wq.to(torch.float32) * s_w[:, None]).t()
    if bias is not None:
        y = y + bias.to(torch.float32)
    return y.to(out_dtype)


def attn_combine_quant(po, pm, pl, *, splits, batch, tokens, heads_q, heads_kv, head_dim, out_dtype=torch.float16,
                       quant=True):
    """Merge of split-KV attention partials + per-token quantiser of the merged row
    (instinctflash/kernels/attention.py:109-145).  Returns (out [B, Tq, Hq, D] in ``out_dtype``,
    codes [Tq, Hq*D] or None, scales [Tq] or None)."""
    block_d = 1 << max(0, (int(head_dim) - 1).bit_length())
    a_po, a_pm, a_pl = _f32(po), _f32(pm), _f32(pl)
    out = np.zeros((batch, tokens, heads_q, head_dim), dtype=np.float32)
    width = heads_q * head_dim
    q = np.zeros((tokens, width), dtype=np.uint8) if quant else None
    qs = np.zeros(tokens, dtype=np.float32) if quant else None
    _lib().oracle_attn_combine_quant(_p(a_po), _p(a_pm), _p(a_pl), int(splits), int(batch), int(tokens), int(heads_q),
                                     int(heads_kv), int(head_dim), block_d, _p(out), _p(q), ctypes.c_int64(width), _p(qs))
    o = torch.from_numpy(out).to(out_dtype)
    return o, (_as_e4m3(q) if quant else None), (torch.from_numpy(qs) if quant else None)
