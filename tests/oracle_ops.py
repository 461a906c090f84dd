"""CPU operator set with the signatures of ``instinctflash_b200.kernels`` (outputs written into
caller-owned tensors), implemented on the CPU oracle.  Lets the host-side drivers (layer stacks,
the tensor-parallel driver) run on CPU under ``gloo`` in the tests.  Test infrastructure only."""
from types import SimpleNamespace

import torch

from oracle import oracle as O

E4M3 = torch.float8_e4m3fn


class CpuFp8Weight:
    def __init__(self, w, scale, bias=None):
        self.w, self.scale, self.bias = w, scale, bias


def gemm(a, w, out):
    out.copy_(O.gemm(a, w.w))
    return out


def gemm_acc(a, w, out):
    out.copy_(O.gemm_acc(a, w.w))
    return out


def row_quant(x, q, q_scale, *, row=None, col=None, bias=None, gelu=False, num_warps=None):
    c, s = O.row_quant(x, row=row, col=col, bias=bias, gelu=gelu)
    q.view(torch.uint8).copy_(c.view(torch.uint8))
    q_scale.copy_(s)


def row_quant_sharded(x, q, q_scale, amax, phase, *, row=None, col=None, bias=None, gelu=False):
    if phase == 1:
        amax.copy_(O.row_quant_sharded(x, None, 1, row=row, col=col, bias=bias, gelu=gelu))
    else:
        c, s = O.row_quant_sharded(x, amax, 2, row=row, col=col, bias=bias, gelu=gelu)
        q.view(torch.uint8).copy_(c.view(torch.uint8))
        q_scale.copy_(s)


def row_max_sharded(x, amax, mirrors=(), *, row=None, col=None, bias=None, gelu=False):
    row_quant_sharded(x, None, None, amax, 1, row=row, col=col, bias=bias, gelu=gelu)
    for t in mirrors:
        t.copy_(amax)


def encode_rowblock_maps(buffers):
    return list(buffers)          # on CPU a "map" is the destination itself


def gemm_rowblocks(a, w, group_rows, maps):
    for g, dst in enumerate(maps):
        gemm_acc(a[group_rows * g: group_rows * (g + 1)], w, dst)


def dequant_rows(x, y, *, row=None, col=None, bias=None, block=None, num_warps=4):
    y.copy_(O.dequant_rows(x, row=row, col=col, bias=bias, out_dtype=y.dtype))


def gated_act_quant(gu, q, q_scale, *, row=None, col=None, act=0, num_warps=None):
    c, s = O.gated_act_quant(gu, row=row, col=col, act=act)
    q.view(torch.uint8).copy_(c.view(torch.uint8))
    q_scale.copy_(s)


def residual_norm_quant(res, *, delta=None, delta_row=None, delta_col=None, bias=None, gate=None, write_res=True,
                        layernorm=False, weight=None, beta=None, mod_scale=None, mod_shift=None, q=None,
                        q_scale=None, y=None, eps=1e-6, num_warps=None, router=None, mod_index=None):
    if delta is not None and delta.ndim == 3:
        # fp32 partial sums of a K-split GEMM: added in plane order, rounded to bf16 like the raw accumulator
        total = delta[0].clone()
        for plane in delta[1:]:
            total = total + plane
        delta = total.to(torch.bfloat16)
    o = O.residual_norm_quant(res, delta=delta, delta_row=delta_row, delta_col=delta_col, bias=bias, gate=gate,
                              write_res=write_res, layernorm=layernorm, weight=weight, beta=beta,
                              mod_scale=mod_scale, mod_shift=mod_shift, mod_index=mod_index, eps=eps,
                              quant=q is not None, y_dtype=None if y is None else y.dtype)
    if delta is not None and write_res:
        res.copy_(o["res"])
    if q is not None:
        q.view(torch.uint8).copy_(o["q"].view(torch.uint8))
        q_scale.copy_(o["qs"])
    if y is not None:
        y.copy_(o["y"])


def residual_norm_quant_peers(res, *, q, q_scale, q_mirrors, q_scale_mirrors, **kw):
    residual_norm_quant(res, q=q, q_scale=q_scale, **kw)
    for t, ts in zip(q_mirrors, q_scale_mirrors):
        t.view(torch.uint8).copy_(q.view(torch.uint8))
        ts.copy_(q_scale)


def ops():
    return SimpleNamespace(gemm=gemm, gemm_acc=gemm_acc, row_quant=row_quant, row_quant_sharded=row_quant_sharded,
                           row_max_sharded=row_max_sharded, gemm_rowblocks=gemm_rowblocks,
                           encode_rowblock_maps=encode_rowblock_maps,
                           residual_norm_quant_peers=residual_norm_quant_peers,
                           dequant_rows=dequant_rows, residual_norm_quant=residual_norm_quant,
                           gated_act_quant=gated_act_quant, GELU_TANH=0, Fp8Weight=CpuFp8Weight)
