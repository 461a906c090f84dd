"""Per-channel e4m3 weights, the raw-accumulator FP8 GEMM and the fused linear.

Drop-in for ``instinctflash/kernels/fp8.py``: ``Fp8Weight`` has the same fields and layout
(``w`` [N, K] e4m3 with K contiguous, ``scale`` [N] float32, ``bias`` [N] float32 or None —
lines 19-27 there), ``quantize_weight`` packs with the same arithmetic (lines 30-37) and
``gemm`` writes ``bf16(sum_k a[m,k] * w[n,k])`` with unit scales (lines 50-53).  The GEMM is the
tcgen05 kernel of ``csrc/gemm_fp8_sm100.cu`` instead of ``torch._scaled_mm``.

``fp8_linear``, ``fp8_linear_residual`` and ``fp8_linear_gated`` are additions: the same GEMM with
the consumer (``dequant_rows`` / the residual part of ``residual_norm_quant`` / the activation part
of ``gated_act_quant``) applied in its epilogue, so the [M, N] raw accumulator never travels
through memory.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib
from ._common import E4M3, launch, ld, rows, same_device, vec

FP8_MAX = 448.0


@dataclass
class Fp8Weight:
    w: torch.Tensor                   # [N, K] e4m3, K contiguous
    scale: torch.Tensor               # [N] float32, per output channel: amax / 448
    bias: torch.Tensor | None = None  # [N] float32

    @property
    def shape(self):
        return tuple(self.w.shape)


def quantize_weight(w: torch.Tensor, bias: torch.Tensor | None = None, device=None) -> Fp8Weight:
    """Pack ``w`` [N, K] (any float dtype) with one scale per output channel on ``device``.

    Load-time work, plain torch: scale = max(|row|, 1e-12) / 448, codes = e4m3_rn(clamp(w / scale)).
    """
    if w.ndim != 2:
        raise ValueError(f"weight must be [N, K], got shape {tuple(w.shape)}")
    target = device if device is not None else w.device
    wf = w.to(device=target, dtype=torch.float32)
    channel_max = wf.abs().amax(dim=1).clamp_min(1e-12)
    scale = channel_max / FP8_MAX
    codes = (wf / scale[:, None]).clamp_(-FP8_MAX, FP8_MAX).to(E4M3).contiguous()
    packed_bias = None
    if bias is not None:
        packed_bias = bias.to(device=wf.device, dtype=torch.float32).contiguous()
    return Fp8Weight(codes, scale.contiguous(), packed_bias)


def _operands(a: torch.Tensor, w: Fp8Weight):
    rows(a, "a", (E4M3,))
    rows(w.w, "w.w", (E4M3,))
    if w.w.device != a.device:
        raise ValueError("activations and weights must be on the same device")
    M, K = a.shape
    N, Kw = w.w.shape
    if K != Kw:
        raise ValueError(f"a is [M, {K}] but the weight is [{N}, {Kw}]")
    if K % 16 or N % 16:
        raise ValueError("FP8 GEMM input/output dimensions must be multiples of 16")
    return M, N, K


def gemm(a: torch.Tensor, w: Fp8Weight, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] (bf16) = a[M, K] (e4m3) @ w.w[N, K]^T, unscaled raw accumulator."""
    M, N, K = _operands(a, w)
    rows(out, "out", (torch.bfloat16,))
    if tuple(out.shape) != (M, N):
        raise ValueError(f"out must be [{M}, {N}], got {tuple(out.shape)}")
    same_device(a, out=out)
    launch("iflb200_gemm_fp8_raw", a, a.data_ptr(), ld(a), w.w.data_ptr(), ld(w.w), M, N, K, out.data_ptr(), ld(out))
    return out


def fp8_linear(a: torch.Tensor, a_scale: torch.Tensor | None, w: Fp8Weight, out: torch.Tensor, *,
               bias: torch.Tensor | None = None, use_weight_bias: bool = True,
               exact: bool = False) -> torch.Tensor:
    """``gemm`` + ``dequant_rows`` in one kernel.

    out[m, n] = out.dtype(fma(r * a_scale[m], w.scale[n], bias[n])) with r the accumulator
    rounded to bf16 first (the reference's memory round trip) unless ``exact``.
    ``a_scale`` is [M] (per token) or a single element (per tensor); ``w.scale`` likewise
    [N] or one element.  ``bias`` overrides ``w.bias`` (float32 or bf16).
    """
    M, N, K = _operands(a, w)
    rows(out, "out", (torch.float32, torch.bfloat16, torch.float16))
    if tuple(out.shape) != (M, N):
        raise ValueError(f"out must be [{M}, {N}], got {tuple(out.shape)}")
    b = bias if bias is not None else (w.bias if use_weight_bias else None)
    if b is not None:
        if b.dtype not in (torch.float32, torch.bfloat16) or b.numel() != N or not b.is_contiguous():
            raise ValueError("bias must be a contiguous float32 or bfloat16 vector of N elements")
    rs = vec(a_scale, "a_scale", None, a.device)
    cs = vec(w.scale, "w.scale", None, a.device)
    if rs is not None and rs.numel() not in (1, M):
        raise ValueError(f"a_scale must have 1 or {M} elements")
    if cs is not None and cs.numel() not in (1, N):
        raise ValueError(f"w.scale must have 1 or {N} elements")
    same_device(a, out=out, bias=b)
    launch("iflb200_fp8_linear", a,
        a.data_ptr(), ld(a), w.w.data_ptr(), ld(w.w), M, N, K,
        _lib.ptr(rs), 0 if (rs is not None and rs.numel() == 1 and M != 1) else 1,
        _lib.ptr(cs), 0 if (cs is not None and cs.numel() == 1 and N != 1) else 1,
        _lib.ptr(b), _lib.dtype_code(b.dtype) if b is not None else _lib.F32,
        _lib.ROUND_EXACT if exact else _lib.ROUND_ENGINE,
        out.data_ptr(), _lib.dtype_code(out.dtype), ld(out))
    return out


def fp8_linear_residual(a: torch.Tensor, a_scale: torch.Tensor, w: Fp8Weight, res: torch.Tensor, *,
                        bias: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                        gate_index: torch.Tensor | None = None) -> torch.Tensor:
    """``gemm`` + the residual part of ``residual_norm_quant`` in one kernel (in place on ``res``).

    res[m, n] += (r * a_scale[m] * w.scale[n] (+ bias[n])) (* gate[idx[m], n]), r the bf16-rounded
    accumulator; stored in ``res``'s dtype (float32, or bf16 for the Wan residual stream).
    """
    M, N, K = _operands(a, w)
    rows(res, "res", (torch.float32, torch.bfloat16))
    if tuple(res.shape) != (M, N):
        raise ValueError(f"res must be [{M}, {N}], got {tuple(res.shape)}")
    rs = vec(a_scale, "a_scale", M, a.device)
    cs = vec(w.scale, "w.scale", N, a.device)
    b = vec(bias, "bias", N, a.device)
    g = vec(gate, "gate", N, a.device)
    if gate_index is not None and (gate_index.dtype != torch.int32 or gate_index.numel() < M):
        raise ValueError("gate_index must be int32 with one entry per row")
    same_device(a, res=res, gate_index=gate_index)
    launch("iflb200_fp8_linear_residual", a,
        a.data_ptr(), ld(a), w.w.data_ptr(), ld(w.w), M, N, K, _lib.ptr(rs), _lib.ptr(cs),
        _lib.ptr(b), _lib.ptr(g), _lib.ptr(gate_index), res.data_ptr(), _lib.dtype_code(res.dtype),
        ld(res))
    return res


def fp8_linear_gated(a: torch.Tensor, a_scale: torch.Tensor, w: Fp8Weight, h: torch.Tensor, amax: torch.Tensor, *,
                     act: int = 0) -> torch.Tensor:
    """``gemm`` on a ``[gate | up]`` weight + the activation part of ``gated_act_quant`` in one kernel.

    ``w.w`` is [2F, K]; ``h`` [M, F] float32 receives ``act(g) * u`` of the dequantised accumulators
    (never rounded to 16 bits, like the reference's registers); ``amax`` [M] float32 must be zero on
    entry and holds each row's maximum of ``|h|`` afterwards.  ``norm.row_quant_from_amax(h, amax,
    q, q_scale)`` finishes the operator: together they write the codes and scales of
    ``gemm`` + ``gated_act_quant`` bit for bit.  ``act``: 0 GELU-tanh, 1 SiLU.
    """
    rows(a, "a", (E4M3,))
    rows(w.w, "w.w", (E4M3,))
    rows(h, "h", (torch.float32,))
    M, K = a.shape
    N2, Kw = w.w.shape
    if K != Kw or N2 % 2:
        raise ValueError(f"a is [M, {K}] but the [gate | up] weight is [{N2}, {Kw}]")
    F = N2 // 2
    if K % 16 or F % 16:
        raise ValueError("FP8 GEMM input/output dimensions must be multiples of 16")
    if tuple(h.shape) != (M, F):
        raise ValueError(f"h must be [{M}, {F}], got {tuple(h.shape)}")
    if act not in (0, 1):
        raise ValueError("act must be GELU_TANH (0) or SILU (1)")
    rs = vec(a_scale, "a_scale", M, a.device)
    cs = vec(w.scale, "w.scale", 2 * F, a.device)
    vec(amax, "amax", M, a.device)
    same_device(a, h=h, w=w.w)
    launch("iflb200_fp8_linear_gated", a, a.data_ptr(), ld(a), w.w.data_ptr(), ld(w.w), M, F, K, _lib.ptr(rs),
           _lib.ptr(cs), int(act), h.data_ptr(), ld(h), amax.data_ptr())
    return h


def partial_splits(M: int, N: int, K: int, sm_count: int = 148) -> int:
    """How many K ranges ``gemm_partials`` should use for a skinny projection: enough (tile, range)
    pairs to occupy the GPU, every range at least four 128-byte K slabs, at most eight planes."""
    if M > 128 or K % 128:
        return 1
    tiles = (N + 63) // 64
    return max(1, min(8, sm_count // max(1, tiles), (K // 128) // 4))


def gemm_partials(a: torch.Tensor, w: Fp8Weight, out: torch.Tensor) -> torch.Tensor:
    """Split-K ``gemm`` for skinny activations: ``out`` [S, M, N] float32 receives the partial sums of
    S K ranges (no scales, no rounding); ``norm.residual_norm_quant(..., delta=out)`` adds the planes
    in order, rounds the sum to bf16 (the raw accumulator's rounding point) and goes on as usual."""
    M, N, K = _operands(a, w)
    if out.dtype != torch.float32 or out.ndim != 3 or tuple(out.shape[1:]) != (M, N) or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous float32 [S, {M}, {N}] tensor")
    if M > 128 or K % 128:
        raise ValueError("gemm_partials is for at most 128 rows and K a multiple of 128")
    same_device(a, out=out)
    launch("iflb200_gemm_fp8_partials", a, a.data_ptr(), ld(a), w.w.data_ptr(), ld(w.w), M, N, K, int(out.shape[0]),
           out.data_ptr(), N)
    return out


def encode_rowblock_maps(buffers) -> torch.Tensor:
    """Device array of tensor maps, one per destination of ``gemm_rowblocks``: ``buffers`` are
    float32 [rows, N] tensors of equal shape with contiguous rows, on this GPU or peer-mapped.  The
    maps hold the buffers' addresses: keep the buffers alive and in place."""
    first = buffers[0]
    host = torch.zeros(len(buffers), 128, dtype=torch.uint8)
    for i, b in enumerate(buffers):
        if b.dtype != torch.float32 or b.ndim != 2 or b.shape != first.shape or b.stride(1) != 1:
            raise ValueError("destinations must be float32 [rows, N] tensors of one shape")
        _lib.check(_lib.lib().iflb200_encode_rowblock_map(b.data_ptr(), int(b.shape[0]), int(b.shape[1]), ld(b),
                                                          host[i].data_ptr()), "encode_rowblock_map")
    return host.to(first.device)


def gemm_rowblocks(a: torch.Tensor, w: Fp8Weight, group_rows: int, maps: torch.Tensor) -> None:
    """K-split linear whose row blocks go to different destinations in one launch: ``a`` [G * group_rows,
    K] e4m3, block g's float32 accumulators (no scales, no rounding) stored through ``maps[g]``
    (``encode_rowblock_maps``).  Tiles of the blocks alternate, so stores towards a peer GPU drain
    under the other tiles' main loops."""
    M, N, K = _operands(a, w)
    G = int(maps.shape[0])
    if maps.dtype != torch.uint8 or maps.ndim != 2 or maps.shape[1] != 128 or not maps.is_contiguous() or maps.data_ptr() % 64:
        raise ValueError("maps must be the device tensor encode_rowblock_maps returned")
    if group_rows * G != M:
        raise ValueError(f"a has {M} rows, expected {G} blocks of {group_rows}")
    same_device(a, maps=maps)
    launch("iflb200_gemm_fp8_rowblocks", a, a.data_ptr(), ld(a), w.w.data_ptr(), ld(w.w), G, int(group_rows), N, K,
           maps.data_ptr())

