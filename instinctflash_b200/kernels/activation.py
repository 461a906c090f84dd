"""Gated MLP activation on a raw accumulator, fused with the per-token quantiser.

Drop-in for ``gated_act_quant`` of ``instinctflash/kernels/activation.py`` (lines 20-56):

    g = gu[m, :F] * row[m] * col[:F]          u = gu[m, F:] * row[m] * col[F:]
    h = act(g) * u                            act in {GELU_TANH, SILU}
    q[m], s[m] = e4m3(h / s[m]), rowmax(|h|) / 448

The hidden activation stays in float32 registers between the activation and the cast, as in
the reference.  The reference's mixture-of-experts helpers in the same file are not part of
the FP8 linear path and are not provided.
"""
from __future__ import annotations

import torch

from .. import _lib
from ._common import E4M3, launch, ld, rows, same_device, vec

GELU_TANH = 0
SILU = 1


def gated_act_quant(gu, q, q_scale, *, row=None, col=None, act=GELU_TANH, num_warps=None):
    rows(gu, "gu", (torch.float32, torch.bfloat16, torch.float16))
    rows(q, "q", (E4M3,))
    M, F2 = gu.shape
    F = F2 // 2
    if F2 % 2:
        raise ValueError("gu must hold the gate and up halves side by side (even width)")
    if F > 16384:
        raise ValueError("gated_act_quant supports hidden widths up to 16384")
    if act not in (GELU_TANH, SILU):
        raise ValueError("act must be GELU_TANH (0) or SILU (1)")
    if tuple(q.shape) != (M, F):
        raise ValueError(f"q must be [{M}, {F}], got {tuple(q.shape)}")
    vec(q_scale, "q_scale", M, gu.device)
    same_device(gu, q=q)
    launch("iflb200_gated_act_quant", gu,
        gu.data_ptr(), _lib.dtype_code(gu.dtype), ld(gu), M, F,
        _lib.ptr(vec(row, "row", M, gu.device)), _lib.ptr(vec(col, "col", 2 * F, gu.device)), int(act),
        q.data_ptr(), ld(q), q_scale.data_ptr())
