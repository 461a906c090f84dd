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

Two transports carry the exchange steps.  ``Comm`` alone: NCCL collectives.  With a ``PeerLink``
(peer-mapped buffers over NVLink): the K-split GEMM's TMA stores write each row block of the fp32
partial straight into plane ``rank`` of the rank that owns those rows, so the transfer rides under
the GEMM; the owner's residual kernel sums the planes in rank order (the reduce-scatter's sum, at the
same place before the bf16 rounding); codes, row scales and row maxima travel as peer stores; three
single-CTA barrier kernels per row-split linear replace five library collectives.
"""
from __future__ import annotations

import os
from types import SimpleNamespace

import torch
import torch.distributed as dist

from .kernels import fp8 as _fp8
from .kernels import norm as _norm
from .kernels._common import launch as _launch
from .stack import StackSpec

E4M3 = torch.float8_e4m3fn


def native_ops() -> SimpleNamespace:
    def gemm_acc(a, w, out):
        """fp32 accumulator of a @ w.w^T (no scales, no rounding): the partial sum of a K shard."""
        return _fp8.fp8_linear(a, None, _fp8.Fp8Weight(w.w, None, None), out, use_weight_bias=False, exact=True)

    return SimpleNamespace(gemm=_fp8.gemm, gemm_acc=gemm_acc, row_quant=_norm.row_quant,
                           row_quant_sharded=_norm.row_quant_sharded, row_max_sharded=_norm.row_max_sharded,
                           gemm_rowblocks=_fp8.gemm_rowblocks, encode_rowblock_maps=_fp8.encode_rowblock_maps,
                           dequant_rows=_norm.dequant_rows, residual_norm_quant=_norm.residual_norm_quant,
                           residual_norm_quant_peers=_norm.residual_norm_quant_peers, Fp8Weight=_fp8.Fp8Weight)


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


def _align(n: int, to: int = 256) -> int:
    return (n + to - 1) // to * to


class PeerLink:
    """Named buffers that every rank of a group can write, and the barrier between the ranks.

    Every rank allocates the same arena (``torch.distributed._symmetric_memory``: one physical
    allocation per GPU, mapped into every process of the group with plain peer mappings -- a
    multicast binding is refused, the data path uses ordinary loads and stores) and carves the
    ``layout`` ({name: (shape, dtype)}) out of it at identical offsets.  ``buffer(r, name)`` is rank
    r's copy as a tensor on this device; ``exchange`` is ``iflb200_peer_exchange``: the barrier
    (bounded wait, status word) and an optional max over the ranks' slots.  One process per GPU."""

    def __init__(self, layout: dict, device, group=None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.dev = torch.device(device)
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.size = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.offsets, at = {}, _align(4 * self.size)        # the flag words come first
        for name, (shape, dtype) in layout.items():
            n = 1
            for d in shape:
                n *= int(d)
            self.offsets[name] = (at, tuple(int(d) for d in shape), dtype)
            at += _align(n * torch.empty((), dtype=dtype).element_size())
        self.nbytes = at
        try:
            symm.set_backend("CUDA")      # driver-level peer mappings; no other library on the data path
        except RuntimeError:
            pass                          # already fixed by an earlier allocation
        self.arena = symm.empty(at, dtype=torch.uint8, device=self.dev)
        self.handle = symm.rendezvous(self.arena, self.group)
        if int(getattr(self.handle, "multicast_ptr", 0) or 0) != 0:
            raise RuntimeError("the symmetric arena was bound to a multicast object; set "
                               "TORCH_SYMM_MEM_DISABLE_MULTICAST=1 before the first rendezvous")
        self.base = [int(x) for x in self.handle.buffer_ptrs]
        self.arena.zero_()
        self.arrival = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self._flag_ptrs = torch.tensor(self.base, dtype=torch.int64, device=self.dev)
        self._views = {}
        torch.cuda.synchronize(self.dev)
        dist.barrier(self.group)      # nobody signals before every rank's flag words are zero

    def buffer(self, r: int, name: str) -> torch.Tensor:
        key = (r, name)
        if key not in self._views:
            at, shape, dtype = self.offsets[name]
            esize = torch.empty((), dtype=dtype).element_size()
            # fp8 is a view of bytes: not every torch build hands out symmetric views of that type
            if dtype == E4M3:
                v = self.handle.get_buffer(r, shape, torch.uint8, at).view(E4M3)
            else:
                v = self.handle.get_buffer(r, shape, dtype, at // esize)
            self._views[key] = v
        return self._views[key]

    def local(self, name: str) -> torch.Tensor:
        return self.buffer(self.rank, name)

    def put(self, name: str, index) -> None:
        """Copy region ``index`` (along the first dimension) of the local buffer into the same
        region of every peer's copy (copy engines over NVLink); an ``exchange`` must follow before
        anyone reads it."""
        src = self.local(name)[index]
        for step in range(1, self.size):
            d = (self.rank + step) % self.size
            self.buffer(d, name)[index].copy_(src)

    def exchange(self, maxima=None) -> None:
        """The barrier.  ``maxima=(name, out)``: afterwards out[i] = max over r of the local ``name``
        buffer [p][n] (slot r written by rank r before it arrived)."""
        max_in = max_out = None
        max_n = 0
        if maxima is not None:
            name, out = maxima
            slots = self.local(name)
            max_in, max_out, max_n = slots.data_ptr(), out.data_ptr(), int(slots.shape[1])
        _launch("iflb200_peer_exchange", self.arrival, self._flag_ptrs.data_ptr(), self.base[self.rank],
                self.arrival.data_ptr(), self.rank, self.size, self.status.data_ptr(), max_in, max_out, max_n)

    def check(self) -> None:
        """Host read of the status word (after a synchronize): raises if a wait ran out."""
        word = int(self.status.item()) & 0xFFFFFFFF
        if word:
            self.status.zero_()
            raise RuntimeError(f"peer barrier timed out: rank {self.rank} never saw arrival {word & 0xFFFF} "
                               f"of rank {(word >> 16) & 0xFF} (status 0x{word:08x})")


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

    @staticmethod
    def peer_layout(spec: StackSpec, size: int) -> dict:
        """The buffers of the peer-memory transport, per rank: `planes` [p][M/p][D] fp32 (plane r =
        rank r's partial sums of this rank's rows), `amax_all` [p][M] (slot r = rank r's local row
        maxima), and the replicated block input `q8` [M][D] / `s0` [M] that every owner fills by rows."""
        M, D = spec.M, spec.hidden
        return {"planes": ((size, M // size, D), torch.float32), "amax_all": ((size, M), torch.float32),
                "q8": ((M, D), E4M3), "s0": ((M,), torch.float32)}

    def __init__(self, spec: StackSpec, weights, device, comm: Comm, ops=None, link=None):
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
        self.link = link if p > 1 else None
        if self.link is not None:
            if (self.link.rank, self.link.size) != (r, p):
                raise ValueError("the peer link and the communicator describe different groups")
            L = self.link
            self.q8, self.s0 = L.local("q8"), L.local("s0")
            peers = [(r + step) % p for step in range(1, p)]
            # block g of a K-shard's rows belongs to rank g: its partial sums go to plane r over there
            self.plane_maps = self.ops.encode_rowblock_maps([L.buffer(d, "planes")[r] for d in range(p)])
            self.amax_mirrors = [L.buffer(d, "amax_all")[r] for d in peers]
            self.q8_mirrors = [L.buffer(d, "q8")[self.rows] for d in peers]
            self.s0_mirrors = [L.buffer(d, "s0")[self.rows] for d in peers]
        else:
            self.q8 = torch.zeros(M, D, dtype=torch.uint8, device=dev).view(E4M3)  # replicated input codes
            self.s0 = torch.zeros(M, dtype=f32, device=dev)                        # and their row scales
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
        if self.link is not None:
            # the owner's rows are already in place locally: push them to the peers and meet
            self.link.put("q8", self.rows)
            self.link.put("s0", self.rows)
            self.link.exchange()
            return
        self.comm.all_gather(self.q8.view(torch.uint8), self.q8_loc.view(torch.uint8))
        self.comm.all_gather(self.s0, self.s0_loc)

    def load(self, x: torch.Tensor, attn: torch.Tensor):
        """x [M, D] replicated hidden states; attn [M, o_in] synthetic attention output (each rank
        uses its column shard, as head-sharded attention would produce)."""
        p, r = self.comm.size, self.comm.rank
        self.res.copy_(x[self.rows])
        w = attn.shape[1] // p
        self.attn = attn[:, w * r: w * (r + 1)].contiguous()
        q, qs = (self.q8[self.rows], self.s0[self.rows]) if self.link is not None else (self.q8_loc, self.s0_loc)
        self.ops.residual_norm_quant(self.res, layernorm=True, q=q, q_scale=qs)
        self._gather_input()

    @property
    def collectives(self):
        return self.peer_collectives if self.link is not None else self.nccl_collectives

    peer_collectives = ("column-split qkv/cross-q/ff1, row-split o/cross-o/ff2 over peer memory (NVLink): the K-split "
                        "GEMM stores its fp32 partial into the row owner's planes, the owner's residual kernel sums "
                        "them; row maxima, codes and row scales as peer stores; three single-CTA barrier kernels per "
                        "row-split linear, no library collective")
    nccl_collectives = ("column-split qkv/cross-q/ff1, row-split o/cross-o/ff2; per row-split linear one all-reduce-max "
                   "of the [M] row maxima, one fp32 reduce-scatter of the [M, D] partial and all-gathers of the "
                   "codes and row scales (NCCL)")

    def comm_bytes_per_step(self) -> float:
        """Bytes each rank sends per pass: per row-split linear 4*M*D*(p-1)/p (reduce-scatter) +
        (M*D + 4*M)*(p-1)/p (all-gathers) + 4*M*(p-1)/p (all-reduce-max, ring)."""
        sp, p = self.spec, self.comm.size
        n_row = 3 if sp.cross else 2
        M, D = sp.M, sp.hidden
        if self.link is not None:   # every rank stores (p-1)/p of its partial and p-1 copies of its rows and maxima
            return sp.layers * n_row * ((4.0 * M * D) * (p - 1) / p + (M * D + 4.0 * M) * (p - 1) / p + 4.0 * M * (p - 1))
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
        if self.link is not None:
            return self._row_linear_peer(x_shard, qk, W, prologue, res_kw)
        o.row_quant_sharded(x_shard, qk, self.s1, self.amax, 1, **prologue)
        self.comm.all_reduce_max(self.amax)
        o.row_quant_sharded(x_shard, qk, self.s1, self.amax, 2, **prologue)
        o.gemm_acc(qk, W, self.part)
        self.comm.reduce_scatter_sum(self.part_loc, self.part)
        o.dequant_rows(self.part_loc, self.delta)            # the bf16 rounding point of the accumulator
        o.residual_norm_quant(self.res, delta=self.delta, delta_row=self.s1[self.rows], delta_col=W.scale,
                              bias=W.bias, layernorm=True, q=self.q8_loc, q_scale=self.s0_loc, **res_kw)
        self._gather_input()

    def _row_linear_peer(self, x_shard, qk, W, prologue, res_kw):
        """The row-split linear over peer memory.  Every buffer a peer writes is read only after the
        barrier that follows the write, and overwritten only after a later barrier that the reader
        reaches after its read (planes: read before the third barrier, written after the first of
        the next linear; maxima slots: read before the second, written after the third; q8 / s0:
        read by the column GEMMs before the first, written after the second)."""
        o, L = self.ops, self.link
        r = L.rank
        o.row_max_sharded(x_shard, L.local("amax_all")[r], self.amax_mirrors, **prologue)
        L.exchange(maxima=("amax_all", self.amax))
        o.row_quant_sharded(x_shard, qk, self.s1, self.amax, 2, **prologue)
        o.gemm_rowblocks(qk, W, self.Ml, self.plane_maps)       # one launch, stores to every owner's planes
        L.exchange()
        o.residual_norm_quant_peers(self.res, delta=L.local("planes"), delta_row=self.s1[self.rows], delta_col=W.scale,
                                    bias=W.bias, layernorm=True, q=self.q8[self.rows], q_scale=self.s0[self.rows],
                                    q_mirrors=self.q8_mirrors, q_scale_mirrors=self.s0_mirrors, **res_kw)
        L.exchange()

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
