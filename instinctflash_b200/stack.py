"""Layer-stack drivers: the reference engines' call order for the FP8 linears of one decoder
layer, chained through a real residual stream, with attention replaced by a fixed synthetic
attention-output buffer.

``gemma`` layers follow instinctflash/engines/pi05/engine.py:199-216 (prefix) and :225-253
(action expert); ``wan`` blocks follow instinctflash/engines/wan_va/engine.py:214-247.  Every
buffer is allocated once (the engines' arena pattern, instinctflash/engines/common.py:7-14);
``forward`` only enqueues kernels on the current stream, so it can be captured in a CUDA graph.
The same driver runs any set of operators with the reference's signatures (``ops`` argument),
so the reference's own kernels can be timed through it.

With this package's operators the driver uses the fused forms by default (``fused="auto"``: for
more than 128 rows): the gated activation is evaluated in the gate_up GEMM's epilogue (``fp8_linear_gated`` +
``row_quant_from_amax`` instead of ``gemm`` + ``gated_act_quant``), bit-identical to the unfused
sequence; ``fused=False`` keeps the reference's three-launch structure per linear.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace

import torch

from .kernels import activation as _act
from .kernels import fp8 as _fp8
from .kernels import norm as _norm

E4M3 = torch.float8_e4m3fn


def native_ops() -> SimpleNamespace:
    return SimpleNamespace(gemm=_fp8.gemm, row_quant=_norm.row_quant, dequant_rows=_norm.dequant_rows,
                           residual_norm_quant=_norm.residual_norm_quant, gated_act_quant=_act.gated_act_quant,
                           GELU_TANH=_act.GELU_TANH, Fp8Weight=_fp8.Fp8Weight,
                           fp8_linear_gated=_fp8.fp8_linear_gated, row_quant_from_amax=_norm.row_quant_from_amax,
                           quant_from_amax=_norm.quant_from_amax,
                           fp8_linear_residual=_fp8.fp8_linear_residual, gemm_partials=_fp8.gemm_partials,
                           partial_splits=_fp8.partial_splits)


@dataclass(frozen=True)
class StackSpec:
    name: str
    kind: str            # "gemma" | "wan"
    layers: int
    M: int
    hidden: int
    ffn: int
    qkv: int
    o_in: int = 0        # width of the attention output fed to the O projection (0: no O projection)
    cross: bool = False  # wan: cross-attention q / o projections
    steps: int = 1       # flow steps (the expert re-reads every weight each step)
    sigma: float = 0.02
    outlier_frac: float = 0.0
    outlier_scale: float = 1.0
    seed: int = 0

    def linears(self):
        """(name, N, K) of the FP8 GEMMs of one layer, in call order."""
        out = [("qkv", self.qkv, self.hidden)]
        if self.o_in:
            out.append(("o", self.hidden, self.o_in))
        if self.cross:
            out += [("cross_q", self.hidden, self.hidden), ("cross_o", self.hidden, self.hidden)]
        if self.kind == "gemma":
            out += [("gate_up", 2 * self.ffn, self.hidden), ("down", self.hidden, self.ffn)]
        else:
            out += [("ff1", self.ffn, self.hidden), ("ff2", self.hidden, self.ffn)]
        return out

    def flops(self) -> float:
        return 2.0 * self.M * sum(n * k for _, n, k in self.linears()) * self.layers * self.steps

    def weight_bytes(self) -> float:
        return float(sum(n * k for _, n, k in self.linears()) * self.layers)


SPECS = {
    # pi05 PaliGemma prefix (Gemma-2B): 18 layers, M = 3*256 image + 48 text tokens
    "c2": StackSpec("c2", "gemma", 18, 816, 2048, 16384, 2560, o_in=2048, outlier_frac=0.01, outlier_scale=20.0, seed=1),
    # pi05 action expert (Gemma-300M shape), 10 flow steps, M = 50 action tokens per episode
    "c3": StackSpec("c3", "gemma", 18, 50, 1024, 4096, 1536, steps=10, seed=2),
    # the reference engine's true expert shapes (fused QKV 2560, O projection 2048 -> 1024)
    "c3ref": StackSpec("c3ref", "gemma", 18, 50, 1024, 4096, 2560, o_in=2048, steps=10, seed=2),
    # LingBot-VA / Wan2.2-5B-shape DiT
    "c4": StackSpec("c4", "wan", 30, 4680, 3072, 14336, 9216, o_in=3072, cross=True, outlier_frac=0.005,
                    outlier_scale=30.0, seed=3),
    # DreamZero / Wan-14B-shape DiT, CFG batch 2 x 8192 tokens
    "c5": StackSpec("c5", "wan", 40, 16384, 5120, 13824, 15360, o_in=5120, sigma=0.015, outlier_frac=0.005,
                    outlier_scale=30.0, seed=4),
}


def small_spec(spec: StackSpec, layers: int = 2, M: int | None = None) -> StackSpec:
    """Same layer geometry, fewer layers / rows: the parity-test size."""
    return StackSpec(**{**spec.__dict__, "layers": layers, "M": M if M is not None else spec.M,
                        "name": spec.name + "_small"})


@dataclass
class LayerWeights:
    w: dict = field(default_factory=dict)   # name -> Fp8Weight-like (w, scale, bias)
    vec: dict = field(default_factory=dict)  # name -> float32 vectors (norm affine, gates, modulation)


def make_weights(spec: StackSpec, device, *, cpu_seeded: bool = False):
    """Random-init e4m3 weights of the spec's shapes, packed per output channel
    (``quantize_weight`` arithmetic).  ``cpu_seeded`` draws every tensor on the CPU generator so
    that a CPU oracle sees identical bits (small stacks); otherwise tensors are drawn on the device."""
    dev = torch.device(device)
    gen = torch.Generator(device="cpu" if cpu_seeded else dev).manual_seed(1000 + spec.seed)
    src = "cpu" if cpu_seeded else dev

    def randn(*shape, scale=1.0):
        return torch.randn(*shape, generator=gen, device=src, dtype=torch.float32) * scale

    layers = []
    for _ in range(spec.layers):
        lw = LayerWeights()
        for name, n, k in spec.linears():
            w = randn(n, k, scale=spec.sigma)
            amax = w.abs().amax(dim=1).clamp_min(1e-12)
            scale = amax / 448.0 if cpu_seeded else amax * torch.tensor(1.0 / 448.0, device=dev)
            q = (w / scale[:, None]).clamp_(-448.0, 448.0).to(E4M3)
            bias = randn(n, scale=0.01) if spec.kind == "wan" else None
            lw.w[name] = _fp8.Fp8Weight(q.to(dev).contiguous(), scale.to(dev).contiguous(),
                                        None if bias is None else bias.to(dev))
            del w
        if spec.kind == "wan":
            D = spec.hidden
            for v in ("norm2_w",):
                lw.vec[v] = (1.0 + randn(D, scale=0.05)).to(dev)
            for v in ("norm2_b", "gate_attn", "gate_ffn", "mod_scale_a", "mod_shift_a", "mod_scale_f", "mod_shift_f"):
                lw.vec[v] = randn(D, scale=0.1).to(dev)
            lw.vec["gate_attn"] = lw.vec["gate_attn"] + 0.5
            lw.vec["gate_ffn"] = lw.vec["gate_ffn"] + 0.5
        layers.append(lw)
    return layers


def make_inputs(spec: StackSpec, device, *, cpu_seeded: bool = True):
    """Hidden states [M, hidden] bf16 ~N(0,1) with outlier channels, and the synthetic attention
    output [M, o_in] that stands in for attention in every layer."""
    gen = torch.Generator(device="cpu").manual_seed(2000 + spec.seed)
    x = torch.randn(spec.M, spec.hidden, generator=gen, dtype=torch.float32)
    if spec.outlier_frac > 0:
        n = max(1, int(round(spec.hidden * spec.outlier_frac)))
        cols = torch.randperm(spec.hidden, generator=gen)[:n]
        x[:, cols] *= spec.outlier_scale
    o_dtype = torch.float16 if spec.kind == "wan" else torch.bfloat16
    attn = torch.randn(spec.M, max(spec.o_in, 16), generator=gen, dtype=torch.float32).to(o_dtype)
    return x.to(torch.bfloat16).to(device), attn.to(device)


class LinearStack:
    """Static buffers + the per-layer call sequence.  ``ops`` supplies the operators."""

    def __init__(self, spec: StackSpec, weights, device, ops=None, *, fused="auto", fuse_residual: bool = False,
                 split_partials: bool = True):
        self.spec, self.weights, self.dev = spec, weights, torch.device(device)
        self.ops = ops or native_ops()
        # fused forms exist only in this package's operator set; "auto" takes the gated epilogue where the
        # GEMM is long enough to hide it (measured: with M = 50 the two-kernel gated form is slower
        # than gemm + gated_act_quant, whose single row kernel costs one short launch)
        if fused == "auto":
            fused = spec.M > 128
        self.fused = bool(fused) and hasattr(self.ops, "fp8_linear_gated")
        self.fuse_residual = fuse_residual and hasattr(self.ops, "fp8_linear_residual")
        # skinny activations: deep, narrow projections (down, o) run split-K over independent CTAs, the
        # residual kernel adds the fp32 partial sums (this package's operators only)
        self.split_partials = (split_partials and spec.kind == "gemma" and spec.M <= 128 and
                               hasattr(self.ops, "gemm_partials"))
        M, D, F = spec.M, spec.hidden, spec.ffn
        dev, bf16, f32 = self.dev, torch.bfloat16, torch.float32
        widest_in = max(k for _, _, k in spec.linears())
        widest_out = max(n for _, n, _ in spec.linears())
        self.q8 = torch.zeros(M * widest_in, dtype=torch.uint8, device=dev).view(E4M3)
        self.raw = torch.zeros(M * widest_out, dtype=bf16, device=dev)
        self.scale = [torch.zeros(M, dtype=f32, device=dev) for _ in range(2)]
        self.res = torch.zeros(M, D, dtype=bf16 if spec.kind == "wan" else f32, device=dev)
        if self.fused and spec.kind == "gemma":
            self.h = torch.zeros(M, F, dtype=f32, device=dev)     # act(g) * u, never rounded to 16 bits
            # row maxima of |h|: two buffers that consecutive gated GEMMs alternate (each quantiser pass
            # clears the one the next GEMM will raise); both zero between forward passes
            self.amax = torch.zeros(2, M, dtype=f32, device=dev)
        if self.split_partials:
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            ks = [k for name, n, k in spec.linears() if n == D and name in ("o", "down")]
            self.splits = {k: self.ops.partial_splits(M, D, k, sms) for k in ks}
            self.part = torch.zeros(max(self.splits.values(), default=1) * M * D, dtype=f32, device=dev)
        self.attn = None
        self.launches_per_forward = 0

    def _q8(self, cols):
        return self.q8[: self.spec.M * cols].view(self.spec.M, cols)

    def _raw(self, cols):
        return self.raw[: self.spec.M * cols].view(self.spec.M, cols)

    def load(self, x: torch.Tensor, attn: torch.Tensor):
        """Start of an inference: residual stream <- x, first producer (norm + quantiser)."""
        self.res.copy_(x)
        self.attn = attn
        self.ops.residual_norm_quant(self.res, layernorm=self.spec.kind == "wan", q=self._q8(self.spec.hidden),
                                     q_scale=self.scale[0])

    def forward(self):
        sp, o, s = self.spec, self.ops, self.scale
        D, F = sp.hidden, sp.ffn
        n = 0
        gated = 0   # gated GEMMs issued so far in this pass
        for _ in range(sp.steps):
            for lw in self.weights:
                W = lw.w
                if sp.kind == "gemma":
                    o.gemm(self._q8(D), W["qkv"], self._raw(sp.qkv)); n += 1
                    if sp.o_in:
                        o.row_quant(self.attn, self._q8(sp.o_in), s[1]); n += 1
                        n += self._residual_linear(self._q8(sp.o_in), s[1], W["o"])
                    if self.fused:
                        cur, nxt = self.amax[gated & 1], self.amax[(gated + 1) & 1]
                        gated += 1
                        o.fp8_linear_gated(self._q8(D), s[0], W["gate_up"], self.h, cur, act=o.GELU_TANH); n += 1
                        o.quant_from_amax(self.h, cur, self._q8(F), s[1], zero=nxt); n += 1
                    else:
                        o.gemm(self._q8(D), W["gate_up"], self._raw(2 * F)); n += 1
                        o.gated_act_quant(self._raw(2 * F), self._q8(F), s[1], row=s[0], col=W["gate_up"].scale,
                                          act=o.GELU_TANH); n += 1
                    n += self._residual_linear(self._q8(F), s[1], W["down"])
                else:
                    V = lw.vec
                    o.gemm(self._q8(D), W["qkv"], self._raw(sp.qkv)); n += 1
                    o.row_quant(self.attn, self._q8(D), s[1]); n += 1
                    o.gemm(self._q8(D), W["o"], self._raw(D)); n += 1
                    o.residual_norm_quant(self.res, delta=self._raw(D), delta_row=s[1], delta_col=W["o"].scale,
                                          bias=W["o"].bias, gate=V["gate_attn"], layernorm=True, weight=V["norm2_w"],
                                          beta=V["norm2_b"], q=self._q8(D), q_scale=s[0]); n += 1
                    if sp.cross:
                        o.gemm(self._q8(D), W["cross_q"], self._raw(D)); n += 1
                        o.row_quant(self.attn, self._q8(D), s[1]); n += 1
                        o.gemm(self._q8(D), W["cross_o"], self._raw(D)); n += 1
                        o.residual_norm_quant(self.res, delta=self._raw(D), delta_row=s[1], delta_col=W["cross_o"].scale,
                                              bias=W["cross_o"].bias, layernorm=True, mod_scale=V["mod_scale_a"],
                                              mod_shift=V["mod_shift_a"], q=self._q8(D), q_scale=s[0]); n += 1
                    o.gemm(self._q8(D), W["ff1"], self._raw(F)); n += 1
                    o.row_quant(self._raw(F), self._q8(F), s[1], row=s[0], col=W["ff1"].scale, bias=W["ff1"].bias,
                                gelu=True); n += 1
                    o.gemm(self._q8(F), W["ff2"], self._raw(D)); n += 1
                    o.residual_norm_quant(self.res, delta=self._raw(D), delta_row=s[1], delta_col=W["ff2"].scale,
                                          bias=W["ff2"].bias, gate=V["gate_ffn"], layernorm=True,
                                          mod_scale=V["mod_scale_f"], mod_shift=V["mod_shift_f"], q=self._q8(D),
                                          q_scale=s[0]); n += 1
        if gated:
            self.amax[(gated - 1) & 1].zero_()   # the last pass's own maxima: both buffers zero again
        self.launches_per_forward = n
        return self.res

    def _residual_linear(self, a, a_scale, w) -> int:
        """res += (a @ w^T) * a_scale * w.scale, then RMS norm + quantiser of the new residual
        stream into q8 / scale[0] (Gemma layers).  Returns the number of launches."""
        o, D = self.ops, self.spec.hidden
        S = self.splits.get(a.shape[1], 1) if self.split_partials else 1
        if S > 1:
            part = self.part[: S * self.spec.M * D].view(S, self.spec.M, D)
            o.gemm_partials(a, w, part)
            o.residual_norm_quant(self.res, delta=part, delta_row=a_scale, delta_col=w.scale,
                                  q=self._q8(D), q_scale=self.scale[0])
        elif self.fuse_residual:
            o.fp8_linear_residual(a, a_scale, w, self.res)
            o.residual_norm_quant(self.res, q=self._q8(D), q_scale=self.scale[0])
        else:
            o.gemm(a, w, self._raw(D))
            o.residual_norm_quant(self.res, delta=self._raw(D), delta_row=a_scale, delta_col=w.scale,
                                  q=self._q8(D), q_scale=self.scale[0])
        return 2

    def capture(self):
        """Warm up on a side stream, then capture ``forward`` into a CUDA graph
        (instinctflash/engines/common.py:34-47)."""
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.forward()
        torch.cuda.current_stream(self.dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward()
        return graph


class HostPipeline:
    """Serving loop around one stack whose inputs arrive in pinned host memory and whose residual
    stream goes back to the host: step i's host-to-device copy runs on a copy stream while step
    i-1 computes, and step i's result leaves on a second copy stream while step i+1 computes (two
    staging buffers each way).  Every step still copies its own input in and its own result out;
    only the waiting is overlapped."""

    def __init__(self, stack, graph, depth: int = 2):
        self.stack, self.graph, self.depth = stack, graph, depth
        dev = stack.dev
        self.dev = dev
        self.h2d, self.d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.x_stage = [torch.empty_like(stack.res) for _ in range(depth)]
        self.out_stage = [torch.empty_like(stack.res) for _ in range(depth)]
        self.x_ready = [torch.cuda.Event() for _ in range(depth)]      # staging input i holds this step's data
        self.x_free = [torch.cuda.Event() for _ in range(depth)]       # the stack has consumed staging input i
        self.out_ready = [torch.cuda.Event() for _ in range(depth)]    # staging output i holds this step's result
        self.out_free = [torch.cuda.Event() for _ in range(depth)]     # staging output i has left for the host
        self.step = 0

    def submit(self, x_host: torch.Tensor, out_host: torch.Tensor, attn: torch.Tensor) -> None:
        """Enqueue one inference: x_host (pinned) in, the residual stream into out_host (pinned).
        Returns at once; ``drain`` waits for everything enqueued so far."""
        i, k = self.step, self.step % self.depth
        main = torch.cuda.current_stream(self.dev)
        with torch.cuda.stream(self.h2d):
            if i >= self.depth:
                self.h2d.wait_event(self.x_free[k])
            self.x_stage[k].copy_(x_host, non_blocking=True)
            self.x_ready[k].record(self.h2d)
        main.wait_event(self.x_ready[k])
        self.stack.load(self.x_stage[k], attn)
        self.x_free[k].record(main)
        self.graph.replay()
        if i >= self.depth:
            main.wait_event(self.out_free[k])
        self.out_stage[k].copy_(self.stack.res, non_blocking=True)
        self.out_ready[k].record(main)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.out_ready[k])
            out_host.copy_(self.out_stage[k], non_blocking=True)
            self.out_free[k].record(self.d2h)
        self.step += 1

    def drain(self) -> None:
        """Make the current stream wait for every copy enqueued so far (no host synchronisation)."""
        main = torch.cuda.current_stream(self.dev)
        main.wait_stream(self.h2d)
        main.wait_stream(self.d2h)


class EpisodeBatch:
    """``episodes`` independent inferences of one stack on one GPU: one ``LinearStack`` each (own
    activations, residual stream and scales) over shared weights, captured as parallel branches
    of ONE CUDA graph, so that the GPU always has several short dependent chains to pick kernels
    from.  Every GEMM keeps the row count of a single episode.  Independent robot episodes are what
    the skinny action-expert configuration shards over GPUs; this is the per-GPU part."""

    def __init__(self, spec: StackSpec, weights, device, episodes: int, **stack_kw):
        self.spec, self.dev = spec, torch.device(device)
        self.stacks = [LinearStack(spec, weights, device, **stack_kw) for _ in range(episodes)]
        self.streams = [torch.cuda.Stream(self.dev) for _ in range(episodes)]
        self.launches_per_forward = 0

    def load(self, x, attn):
        xs = x if isinstance(x, (list, tuple)) else [x] * len(self.stacks)
        for st, xi in zip(self.stacks, xs):
            st.load(xi, attn)

    def forward(self):
        """Fork every episode onto its own stream, join on the current one."""
        main = torch.cuda.current_stream(self.dev)
        for st, side in zip(self.stacks, self.streams):
            side.wait_stream(main)
            with torch.cuda.stream(side):
                st.forward()
        for side in self.streams:
            main.wait_stream(side)
        self.launches_per_forward = sum(st.launches_per_forward for st in self.stacks)
        return [st.res for st in self.stacks]

    def capture(self):
        warm = torch.cuda.Stream(self.dev)
        warm.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(warm):
            for _ in range(2):
                self.forward()
        torch.cuda.current_stream(self.dev).wait_stream(warm)
        torch.cuda.synchronize(self.dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward()
        return graph
