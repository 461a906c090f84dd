"""Tensor-parallel driver for the Wan-shape DiT linears (column-split N for qkv / cross-q / ff1,
row-split K for o / cross-o / ff2), one process per GPU, NCCL collectives over NVLink.

The reference has nothing distributed (it guards world_size == 1:
instinctflash/descriptors/deployment.py:32-37, instinctflash/runtime/wan_va_engine_build.py:72-74);
the oracle of this path is the single-GPU stack of the same build (``stack.LinearStack``):

* weights are packed first and sharded second, so every shard keeps the scales of the full matrix;
* column-split GEMMs produce bit-identical columns (the K loop order depends on K alone);
* a per-token quantiser over column-sharded rows runs in two phases around one all-reduce-max of
  the ``[M]`` row maxima, so the e4m3 codes and scales equal the single-GPU ones bit for bit;
* row-split GEMMs write their fp32 partial accumulators, which are reduce-scattered (summed) in
  fp32 BEFORE the bf16 rounding point; only these sums differ from the single-GPU accumulator
  (summation order), within the GEMM tolerance;
* the residual stream is sharded by rows after the reduce-scatter; the next block's replicated
  input (codes + row scales) is rebuilt with an all-gather.

Bytes per row-split linear and rank: reduce-scatter 4*M*D*(p-1)/p in + all-gather (M*D + 4*M)*(p-1)/p.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.distributed as dist

from .kernels import fp8 as _fp8
from .kernels import norm as _norm
from .stack import StackSpec

E4M3 = torch.float8_e4m3fn


def native_ops() -> SimpleNamespace:
    def gemm_acc(a, w, out):
        """fp32 accumulator of a @ w.w^T (no scales, no rounding): the partial sum of a K shard."""
        return _fp8.fp8_linear(a, None, _fp8.Fp8Weight(w.w, None, None), out, use_weight_bias=False, exact=True)

    return SimpleNamespace(gemm=_fp8.gemm, gemm_acc=gemm_acc, row_quant=_norm.row_quant,
                           row_quant_sharded=_norm.row_quant_sharded,
                           dequant_rows=_norm.dequant_rows, residual_norm_quant=_norm.residual_norm_quant,
                           Fp8Weight=_fp8.Fp8Weight)


class Comm:
    """The three collectives the path needs, on a torch.distributed group."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    @classmethod
    def single(cls):
        """A group of one without a process group (every collective is a copy or nothing)."""
        self = cls.__new__(cls)
        self.group, self.rank, self.size = None, 0, 1
        return self

    def all_reduce_max(self, t):
        if self.size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    def reduce_scatter_sum(self, out, inp):
        if self.size == 1:
            out.copy_(inp)
        else:
            dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def all_gather(self, out, inp):
        if self.size == 1:
            out.copy_(inp)
        else:
            dist.all_gather_into_tensor(out, inp, group=self.group)
        return out


def shard_columns(w, rank: int, size: int):
    """Rows [N/p*r, N/p*(r+1)) of a packed weight (output channels): N-split."""
    N = w.w.shape[0]
    if N % (16 * size):
        raise ValueError(f"N={N} must be a multiple of 16*{size} for a column split")
    lo, hi = N // size * rank, N // size * (rank + 1)
    return _fp8.Fp8Weight(w.w[lo:hi].contiguous(), w.scale[lo:hi].contiguous(),
                          None if w.bias is None else w.bias[lo:hi].contiguous())


def shard_rows(w, rank: int, size: int):
    """Columns [K/p*r, K/p*(r+1)) of a packed weight (input features): K-split.  Scale and bias
    belong to the output channels and stay whole."""
    K = w.w.shape[1]
    if K % (16 * size):
        raise ValueError(f"K={K} must be a multiple of 16*{size} for a row split")
    lo, hi = K // size * rank, K // size * (rank + 1)
    return _fp8.Fp8Weight(w.w[:, lo:hi].contiguous(), w.scale, w.bias)


class WanTPStack:
    """``stack.LinearStack`` for ``kind == "wan"`` specs, tensor parallel over ``comm``."""

    COLUMN = ("qkv", "cross_q", "ff1")
    ROW = ("o", "cross_o", "ff2")

    def __init__(self, spec: StackSpec, weights, device, comm: Comm, ops=None):
        if spec.kind != "wan":
            raise ValueError("tensor parallelism is defined for the Wan-shape stacks")
        p = comm.size
        if spec.M % p:
            raise ValueError(f"M={spec.M} must be divisible by the group size {p}")
        self.spec, self.dev, self.comm = spec, torch.device(device), comm
        self.ops = ops or native_ops()
        r = comm.rank
        self.layers = []
        for lw in weights:
            W = {}
            for name, w in lw.w.items():
                W[name] = shard_columns(w, r, p) if name in self.COLUMN else shard_rows(w, r, p)
            self.layers.append(SimpleNamespace(w=W, vec=lw.vec))
        M, D, F = spec.M, spec.hidden, spec.ffn
        Ml = M // p
        dev, f32, bf16 = self.dev, torch.float32, torch.bfloat16
        self.Ml, self.rows = Ml, slice(Ml * r, Ml * (r + 1))
        self.q8 = torch.zeros(M, D, dtype=torch.uint8, device=dev).view(E4M3)      # replicated input codes
        self.s0 = torch.zeros(M, dtype=f32, device=dev)                            # and their row scales
        self.q8_loc = torch.zeros(Ml, D, dtype=torch.uint8, device=dev).view(E4M3)
        self.s0_loc = torch.zeros(Ml, dtype=f32, device=dev)
        self.qk = torch.zeros(M * max(D, F) // p, dtype=torch.uint8, device=dev).view(E4M3)  # K-shard codes
        self.s1 = torch.zeros(M, dtype=f32, device=dev)
        self.amax = torch.zeros(M, dtype=f32, device=dev)
        self.raw = torch.zeros(M * max(spec.qkv, F) // p, dtype=bf16, device=dev)   # column-shard raw accumulators
        self.part = torch.zeros(M, D, dtype=f32, device=dev)                        # fp32 partial of a K shard
        self.part_loc = torch.zeros(Ml, D, dtype=f32, device=dev)
        self.delta = torch.zeros(Ml, D, dtype=bf16, device=dev)
        self.res = torch.zeros(Ml, D, dtype=bf16, device=dev)                       # residual stream, local rows
        self.attn = None

    def _raw(self, cols):
        return self.raw[: self.spec.M * cols].view(self.spec.M, cols)

    def _qk(self, cols):
        return self.qk[: self.spec.M * cols].view(self.spec.M, cols)

    def _gather_input(self):
        self.comm.all_gather(self.q8.view(torch.uint8), self.q8_loc.view(torch.uint8))
        self.comm.all_gather(self.s0, self.s0_loc)

    def load(self, x: torch.Tensor, attn: torch.Tensor):
        """x [M, D] replicated hidden states; attn [M, o_in] synthetic attention output (each rank
        uses its column shard, as head-sharded attention would produce)."""
        p, r = self.comm.size, self.comm.rank
        self.res.copy_(x[self.rows])
        w = attn.shape[1] // p
        self.attn = attn[:, w * r: w * (r + 1)].contiguous()
        self.ops.residual_norm_quant(self.res, layernorm=True, q=self.q8_loc, q_scale=self.s0_loc)
        self._gather_input()

    collectives = ("column-split qkv/cross-q/ff1, row-split o/cross-o/ff2; per row-split linear one all-reduce-max "
                   "of the [M] row maxima, one fp32 reduce-scatter of the [M, D] partial and all-gathers of the "
                   "codes and row scales (NCCL)")

    def comm_bytes_per_step(self) -> float:
        """Bytes each rank sends per pass: per row-split linear 4*M*D*(p-1)/p (reduce-scatter) +
        (M*D + 4*M)*(p-1)/p (all-gathers) + 4*M*(p-1)/p (all-reduce-max, ring)."""
        sp, p = self.spec, self.comm.size
        n_row = 3 if sp.cross else 2
        M, D = sp.M, sp.hidden
        return sp.layers * n_row * ((4.0 * M * D) + (M * D + 4.0 * M) + 4.0 * M) * (p - 1) / p

    def _row_linear(self, x_shard, W, prologue, res_kw):
        """Quantise the local column shard with global row scales, K-split GEMM, fp32
        reduce-scatter, bf16 rounding, residual + norm + quantiser on the local rows, all-gather.
        A group of one has nothing to exchange: one quantiser pass, the raw bf16 accumulator straight
        from the GEMM, the residual kernel writing the replicated buffers (the single-GPU sequence)."""
        o, sp = self.ops, self.spec
        Kl = x_shard.shape[1]
        qk = self._qk(Kl)
        if self.comm.size == 1 and hasattr(o, "row_quant"):
            o.row_quant(x_shard, qk, self.s1, **prologue)
            o.gemm(qk, W, self.delta)
            o.residual_norm_quant(self.res, delta=self.delta, delta_row=self.s1, delta_col=W.scale, bias=W.bias,
                                  layernorm=True, q=self.q8, q_scale=self.s0, **res_kw)
            return
        o.row_quant_sharded(x_shard, qk, self.s1, self.amax, 1, **prologue)
        self.comm.all_reduce_max(self.amax)
        o.row_quant_sharded(x_shard, qk, self.s1, self.amax, 2, **prologue)
        o.gemm_acc(qk, W, self.part)
        self.comm.reduce_scatter_sum(self.part_loc, self.part)
        o.dequant_rows(self.part_loc, self.delta)            # the bf16 rounding point of the accumulator
        o.residual_norm_quant(self.res, delta=self.delta, delta_row=self.s1[self.rows], delta_col=W.scale,
                              bias=W.bias, layernorm=True, q=self.q8_loc, q_scale=self.s0_loc, **res_kw)
        self._gather_input()

    def forward(self):
        sp, o = self.spec, self.ops
        D, F, p = sp.hidden, sp.ffn, self.comm.size
        for lw in self.layers:
            W, V = lw.w, lw.vec
            o.gemm(self.q8, W["qkv"], self._raw(sp.qkv // p))
            self._row_linear(self.attn, W["o"], {}, dict(gate=V["gate_attn"], weight=V["norm2_w"], beta=V["norm2_b"]))
            if sp.cross:
                o.gemm(self.q8, W["cross_q"], self._raw(D // p))
                self._row_linear(self.attn, W["cross_o"], {}, dict(mod_scale=V["mod_scale_a"], mod_shift=V["mod_shift_a"]))
            raw_ff = self._raw(F // p)
            o.gemm(self.q8, W["ff1"], raw_ff)
            self._row_linear(raw_ff, W["ff2"], dict(row=self.s0, col=W["ff1"].scale, bias=W["ff1"].bias, gelu=True),
                             dict(gate=V["gate_ffn"], mod_scale=V["mod_scale_f"], mod_shift=V["mod_shift_f"]))
        return self.res

    def gather_residual(self):
        """The full residual stream [M, D] (for comparison with the single-GPU stack)."""
        full = torch.empty(self.spec.M, self.spec.hidden, dtype=self.res.dtype, device=self.dev)
        self.comm.all_gather(full, self.res)
        return full
