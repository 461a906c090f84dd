"""Whole-stack persistent execution of the skinny-M action-expert loop (one cooperative launch).

Builds the operator program that ``libiflb200.so``'s ``iflb200_stack_run`` interprets, for the
Gemma-shape expert layers of ``stack.LinearStack`` without an O projection (the benchmark's
expert configuration): per layer and flow step

    qkv GEMM            raw[M, qkv]          (consumer outside this path)
    gate_up GEMM        raw[M, 2F]
    gated_act_quant     -> codes [M, F], row scales
    down GEMM           fp32 partials [split_k][M, D]  (or raw bf16 with split_k = 1)
    residual + RMS norm + quantiser -> codes [M, D], row scales

i.e. the call sequence of instinctflash/engines/pi05/engine.py:225-253 with attention left out.
Operator arithmetic is that of the stand-alone kernels; with ``split_k == 1`` the result is
bit-identical to ``LinearStack`` on the same weights.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .kernels import norm as _norm
from .kernels._common import launch
from .stack import StackSpec

E4M3 = torch.float8_e4m3fn

OP_DTYPE = np.dtype([
    ("type", "<i4"), ("wait_bar", "<i4"), ("arrive_bar", "<i4"), ("tile_offset", "<i4"),
    ("N", "<i4"), ("K", "<i4"), ("split_k", "<i4"), ("act", "<i4"),
    ("tm_a", "<i4"), ("tm_w", "<i4"), ("pad0", "<i4"), ("pad1", "<i4"),
    ("out", "<u8"), ("in", "<u8"), ("row_scale", "<u8"), ("col_scale", "<u8"), ("out_scale", "<u8"), ("res", "<u8"),
    ("ld_out", "<i8"), ("ld_in", "<i8"), ("eps", "<f4"), ("pad2", "<i4"), ("aux", "<u8"),
])
assert OP_DTYPE.itemsize == 128
GEMM, GATED, RESNORM, GEMM_GATED, ENCODE = 1, 2, 3, 4, 5


class PersistentExpertStack:
    def __init__(self, spec: StackSpec, weights, device, *, down_split_k: int | None = None,
                 gated_in_gemm: bool = True):
        if spec.kind != "gemma" or spec.o_in:
            raise ValueError("the persistent stack covers Gemma-shape expert layers without an O projection")
        if spec.M > 128:
            raise ValueError("the persistent stack is for skinny activations (M <= 128)")
        if spec.hidden % 128 or spec.ffn % 128:
            raise ValueError("the persistent stack maps its operands in 128-byte K slabs: hidden and ffn must be multiples of 128")
        if spec.ffn > 8192 or spec.hidden > 8192:
            raise ValueError("row operators of the persistent stack hold at most 8192 columns")
        lib = _lib.lib()
        self.lib, self.spec, self.weights = lib, spec, weights
        self.dev = torch.device(device)
        dev, f32, bf16 = self.dev, torch.float32, torch.bfloat16
        M, D, F = spec.M, spec.hidden, spec.ffn
        k_steps = (F + 127) // 128
        self.sms = sms = torch.cuda.get_device_properties(dev).multi_processor_count
        if down_split_k is None:
            # enough work items to occupy the SMs: (D / 64) column tiles x split_k
            down_split_k = max(1, min(k_steps, 9, sms // max(1, (D + 63) // 64)))
        if not 1 <= down_split_k <= k_steps:
            raise ValueError("every K split needs at least one 128-byte step")
        self.split_k = down_split_k
        # gated activation in the gate_up GEMM's epilogue (h in fp32 + row maxima, then a short
        # quantiser pass shared by all SMs) instead of a one-row-per-CTA gated_act_quant pass
        self.gated_in_gemm = bool(gated_in_gemm)
        self.h = torch.zeros(M, F, dtype=f32, device=dev)
        self.amax = torch.zeros(M, dtype=f32, device=dev)
        self.q8 = torch.zeros(M, D, dtype=torch.uint8, device=dev).view(E4M3)
        self.q8f = torch.zeros(M, F, dtype=torch.uint8, device=dev).view(E4M3)
        self.s0 = torch.zeros(M, dtype=f32, device=dev)
        self.s1 = torch.zeros(M, dtype=f32, device=dev)
        self.raw_qkv = torch.zeros(M, spec.qkv, dtype=bf16, device=dev)
        self.raw_gu = torch.zeros(M, 2 * F, dtype=bf16, device=dev)
        self.down_out = (torch.zeros(down_split_k, M, D, dtype=f32, device=dev) if down_split_k > 1
                         else torch.zeros(M, D, dtype=bf16, device=dev))
        self.res = torch.zeros(M, D, dtype=f32, device=dev)
        self.status = torch.zeros(2, dtype=torch.int32, device=dev)
        self._build_program()

    # ------------------------------------------------------------------------------------
    def _encode_map(self, t: torch.Tensor, box_rows: int) -> bytes:
        buf = (ctypes.c_uint8 * 128)()
        st = self.lib.iflb200_encode_operand_map(buf, t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows)
        _lib.check(st, "encode_operand_map")
        return bytes(buf)

    def _build_program(self):
        sp, lib = self.spec, self.lib
        M, D, F = sp.M, sp.hidden, sp.ffn
        a_rows = lib.iflb200_stack_activation_box_rows(M)
        w_rows = lib.iflb200_stack_weight_box_rows()
        maps = [self._encode_map(self.q8, a_rows), self._encode_map(self.q8f, a_rows)]
        ops = []
        n_bar = 0
        prev = -1
        qkv_items = (sp.qkv + w_rows - 1) // w_rows
        layer_base = []
        for lw in self.weights:   # one tensor map per weight matrix, shared by all flow steps
            layer_base.append(len(maps))
            for name in ("qkv", "gate_up", "down"):
                if name == "gate_up" and self.gated_in_gemm:
                    buf = (ctypes.c_uint8 * 128)()
                    t = lw.w[name].w
                    _lib.check(lib.iflb200_encode_gated_weight_map(buf, t.data_ptr(), F, t.shape[1], t.stride(0)),
                               "encode_gated_weight_map")
                    maps.append(bytes(buf))
                else:
                    maps.append(self._encode_map(lw.w[name].w, w_rows))
        for _ in range(sp.steps):
            for li, lw in enumerate(self.weights):
                W = lw.w
                base = layer_base[li]
                b1, b2, b3, b4 = n_bar, n_bar + 1, n_bar + 2, n_bar + 3
                n_bar += 4
                ops.append(dict(type=GEMM, wait_bar=prev, arrive_bar=-1, tile_offset=0, N=sp.qkv, K=D, split_k=1,
                                tm_a=0, tm_w=base, out=self.raw_qkv.data_ptr(), ld_out=sp.qkv))
                if self.gated_in_gemm:
                    parts = max(1, self.sms // max(1, M))
                    ops.append(dict(type=GEMM_GATED, wait_bar=prev, arrive_bar=b1, tile_offset=qkv_items, N=F, K=D,
                                    split_k=1, act=0, tm_a=0, tm_w=base + 1, out=self.h.data_ptr(), ld_out=F,
                                    row_scale=self.s0.data_ptr(), col_scale=W["gate_up"].scale.data_ptr(),
                                    aux=self.amax.data_ptr()))
                    ops.append(dict(type=ENCODE, wait_bar=b1, arrive_bar=b2, N=F, split_k=parts, out=self.q8f.data_ptr(),
                                    ld_out=F, **{"in": self.h.data_ptr()}, ld_in=F, out_scale=self.s1.data_ptr(),
                                    aux=self.amax.data_ptr()))
                else:
                    ops.append(dict(type=GEMM, wait_bar=prev, arrive_bar=b1, tile_offset=qkv_items, N=2 * F, K=D, split_k=1,
                                    tm_a=0, tm_w=base + 1, out=self.raw_gu.data_ptr(), ld_out=2 * F))
                    ops.append(dict(type=GATED, wait_bar=b1, arrive_bar=b2, N=F, act=0, out=self.q8f.data_ptr(), ld_out=F,
                                    **{"in": self.raw_gu.data_ptr()}, ld_in=2 * F, row_scale=self.s0.data_ptr(),
                                    col_scale=W["gate_up"].scale.data_ptr(), out_scale=self.s1.data_ptr()))
                ops.append(dict(type=GEMM, wait_bar=b2, arrive_bar=b3, tile_offset=0, N=D, K=F, split_k=self.split_k,
                                tm_a=1, tm_w=base + 2, out=self.down_out.data_ptr(), ld_out=D))
                ops.append(dict(type=RESNORM, wait_bar=b3, arrive_bar=b4, N=D, split_k=self.split_k,
                                out=self.q8.data_ptr(), ld_out=D, **{"in": self.down_out.data_ptr()}, ld_in=D,
                                row_scale=self.s1.data_ptr(), col_scale=W["down"].scale.data_ptr(),
                                out_scale=self.s0.data_ptr(), res=self.res.data_ptr(), eps=1e-6,
                                aux=self.amax.data_ptr() if self.gated_in_gemm else 0))
                prev = b4
        arr = np.zeros(len(ops), dtype=OP_DTYPE)
        for i, op in enumerate(ops):
            for k, v in op.items():
                arr[k][i] = v
        self.num_ops, self.num_bars = len(ops), n_bar
        self.launches_per_forward = 1
        dev = self.dev
        self.d_ops = torch.from_numpy(arr.view(np.uint8).copy()).to(dev)
        raw = np.frombuffer(b"".join(maps), dtype=np.uint8).copy()
        # 64-byte alignment of the tensor-map array: torch allocations are 256-byte aligned
        self.d_maps = torch.from_numpy(raw).to(dev)
        assert self.d_maps.data_ptr() % 64 == 0
        self.d_bars = torch.zeros(max(1, n_bar), dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------------------------
    def load(self, x: torch.Tensor):
        """Residual stream <- x [M, hidden]; first producer (RMS norm + quantiser)."""
        self.res.copy_(x)
        _norm.residual_norm_quant(self.res, q=self.q8, q_scale=self.s0)

    def forward(self):
        launch("iflb200_stack_run", self.res, self.d_ops.data_ptr(), self.num_ops, self.d_maps.data_ptr(),
               self.d_bars.data_ptr(), self.num_bars, self.spec.M, self.status.data_ptr())
        return self.res

    def timeout_record(self) -> int:
        return int(self.status[0].item())
