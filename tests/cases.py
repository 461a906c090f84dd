"""Seeded synthetic inputs shared by the golden-vector generators and the parity tests.

Every tensor is drawn on the CPU from ``torch.Generator().manual_seed(seed)`` in float32 and
then cast, so the CPU oracle, the GPU kernels and the recorded reference outputs all see the
same bits.  Shapes and value distributions are those of the five benchmark configurations
(activations ~N(0,1) with a few outlier channels, weights ~N(0, sigma)).
"""
from __future__ import annotations

import torch


def gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def activations(M: int, K: int, seed: int, *, outlier_frac: float = 0.0, outlier_scale: float = 1.0,
                dtype=torch.bfloat16) -> torch.Tensor:
    g = gen(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    if outlier_frac > 0:
        n = max(1, int(round(K * outlier_frac)))
        cols = torch.randperm(K, generator=g)[:n]
        x[:, cols] *= outlier_scale
    return x.to(dtype)


def weights(N: int, K: int, seed: int, sigma: float = 0.02) -> torch.Tensor:
    return torch.randn(N, K, generator=gen(seed), dtype=torch.float32) * sigma


def vector(n: int, seed: int, *, lo=None, hi=None, sigma: float = 1.0) -> torch.Tensor:
    g = gen(seed)
    if lo is not None:
        return torch.rand(n, generator=g, dtype=torch.float32) * (hi - lo) + lo
    return torch.randn(n, generator=g, dtype=torch.float32) * sigma


# (name, M, K) row-quantiser cases: every distinct activation shape of configs C1..C5 at a row
# count the oracle finishes in seconds, plus ragged / tiny / maximum-width edges.
ROW_QUANT_CASES = [
    ("c1", 64, 1024, dict()),
    ("c2_hidden", 816, 2048, dict(outlier_frac=0.01, outlier_scale=20.0)),
    ("c2_ffn", 96, 16384, dict(outlier_frac=0.01, outlier_scale=20.0)),
    ("c3_hidden", 50, 1024, dict()),
    ("c3_ffn", 50, 4096, dict()),
    ("c4_hidden", 300, 3072, dict(outlier_frac=0.005, outlier_scale=30.0)),
    ("c4_ffn", 120, 14336, dict(outlier_frac=0.005, outlier_scale=30.0)),
    ("c5_hidden", 200, 5120, dict(outlier_frac=0.005, outlier_scale=30.0)),
    ("c5_ffn", 100, 13824, dict(outlier_frac=0.005, outlier_scale=30.0)),
    ("one_row", 1, 16, dict()),
    ("ragged", 7, 1000, dict()),
    ("odd_width", 33, 1152, dict()),
    ("tiny_values", 5, 256, dict()),
    ("zeros", 3, 128, dict()),
]

# (name, M, N, K, sigma, act kwargs): per-linear GEMM parity cases at oracle-friendly sizes.
GEMM_CASES = [
    ("c1", 64, 4096, 1024, 0.02, dict()),
    ("c2_qkv", 816, 2560, 2048, 0.02, dict(outlier_frac=0.01, outlier_scale=20.0)),
    ("c2_o", 816, 2048, 2048, 0.02, dict(outlier_frac=0.01, outlier_scale=20.0)),
    ("c2_gate_up_slice", 816, 1024, 2048, 0.02, dict(outlier_frac=0.01, outlier_scale=20.0)),
    ("c2_down_slice", 200, 2048, 16384, 0.02, dict(outlier_frac=0.01, outlier_scale=20.0)),
    ("c3_qkv", 50, 1536, 1024, 0.02, dict()),
    ("c3_gate_up", 50, 8192, 1024, 0.02, dict()),
    ("c3_down", 50, 1024, 4096, 0.02, dict()),
    ("c3_ref_qkv", 50, 2560, 1024, 0.02, dict()),
    ("c3_ref_o", 50, 1024, 2048, 0.02, dict()),
    ("c4_qkv_slice", 520, 1024, 3072, 0.02, dict(outlier_frac=0.005, outlier_scale=30.0)),
    ("c4_ff2_slice", 260, 3072, 14336, 0.02, dict(outlier_frac=0.005, outlier_scale=30.0)),
    ("c5_ff1_slice", 384, 1024, 5120, 0.015, dict(outlier_frac=0.005, outlier_scale=30.0)),
    ("tiny", 1, 16, 16, 0.5, dict()),
    ("tail_k", 7, 768, 784, 0.05, dict()),
    ("tail_n", 130, 272, 256, 0.05, dict()),
    ("siglip", 40, 1152, 4304, 0.02, dict()),
]


def tiny_values(M, K, seed):
    return (torch.randn(M, K, generator=gen(seed)) * 1e-12).to(torch.bfloat16)


def row_quant_input(name, M, K, kw, seed):
    if name == "tiny_values":
        return tiny_values(M, K, seed)
    if name == "zeros":
        return torch.zeros(M, K, dtype=torch.bfloat16)
    return activations(M, K, seed, **kw)


# ---------------------------------------------------------------------------------------------
# Input builders per operator family.  Each yields (name, dict of CPU tensors / flags).
# ---------------------------------------------------------------------------------------------
def row_quant_cases():
    for i, (name, M, K, kw) in enumerate(ROW_QUANT_CASES):
        yield name, dict(x=row_quant_input(name, M, K, kw, 100 + i))
    yield "fp16_in", dict(x=activations(77, 3072, 150, dtype=torch.float16))
    yield "fp32_in", dict(x=activations(19, 2048, 151, dtype=torch.float32))


def raw_like(M, D, seed, spread=300.0):
    """A bf16 tensor that looks like a raw FP8-GEMM accumulator (values up to a few thousand)."""
    return (activations(M, D, seed, dtype=torch.float32) * spread).to(torch.bfloat16)


def prologue_cases():
    table = [("ff1_gelu", 120, 14336, True, True), ("scaled", 64, 2048, False, False),
             ("scaled_bias", 50, 1536, False, True)]
    for j, (name, M, K, gelu, use_bias) in enumerate(table):
        yield name, dict(x=raw_like(M, K, 200 + j), row=vector(M, 210 + j, lo=0.001, hi=0.02),
                         col=vector(K, 220 + j, lo=0.0001, hi=0.001),
                         bias=vector(K, 230 + j, sigma=0.1) if use_bias else None, gelu=gelu)


def gated_cases():
    for j, (name, M, F) in enumerate([("c2", 96, 16384), ("c3", 50, 4096), ("small", 9, 4096), ("ragged", 5, 1000)]):
        for act, aname in ((0, "gelu"), (1, "silu")):
            yield f"{name}_{aname}", dict(gu=raw_like(M, 2 * F, 300 + j, 200.0), row=vector(M, 310 + j, lo=0.001, hi=0.02),
                                          col=vector(2 * F, 320 + j, lo=0.0005, hi=0.002), act=act)


def dequant_cases():
    table = [("c1_bf16", 64, 4096, torch.bfloat16), ("f32_out", 50, 2560, torch.float32),
             ("f16_out", 33, 1152, torch.float16)]
    for j, (name, M, D, odt) in enumerate(table):
        yield name, dict(x=raw_like(M, D, 400 + j), row=vector(M, 410 + j, lo=0.001, hi=0.02),
                         col=vector(D, 420 + j, lo=0.0001, hi=0.001), bias=vector(D, 430 + j, sigma=0.01),
                         out_dtype=odt)


def resnorm_cases():
    table = [("pi05_prefix", 96, 2048, torch.float32, False, False, False, False, False, False),
             ("pi05_expert", 50, 1024, torch.float32, False, True, False, False, True, False),
             ("wan", 64, 3072, torch.bfloat16, True, True, True, True, True, True),
             ("bias_nogate", 33, 1152, torch.float32, True, False, True, True, False, False)]
    for j, (name, M, D, rdt, use_bias, use_gate, ln, affine, adaptive, idx) in enumerate(table):
        ntab = 3 if idx else 1

        def tab(seed, **kw):
            t = vector(ntab * D, seed, **kw)
            return t.view(ntab, D) if idx else t

        yield name, dict(
            res=activations(M, D, 500 + j, dtype=torch.float32).to(rdt), delta=raw_like(M, D, 510 + j),
            delta_row=vector(M, 520 + j, lo=0.001, hi=0.02), delta_col=vector(D, 530 + j, lo=0.0001, hi=0.001),
            bias=vector(D, 540 + j, sigma=0.05) if use_bias else None,
            gate=tab(550 + j, sigma=0.5) if use_gate else None, layernorm=ln,
            weight=vector(D, 560 + j, lo=0.5, hi=1.5) if affine else None,
            beta=vector(D, 570 + j, sigma=0.1) if affine else None,
            mod_scale=tab(580 + j, sigma=0.1) if adaptive else None,
            mod_shift=tab(590 + j, sigma=0.1) if adaptive else None,
            mod_index=(torch.arange(M, dtype=torch.int32) % ntab) if idx else None)


def pack_weight_cpu(wf: torch.Tensor):
    """Per-channel pack with CPU arithmetic (true division), the form every arm is fed."""
    amax = wf.abs().amax(dim=1).clamp_min(1e-12)
    scale = amax / 448.0
    q = (wf / scale[:, None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.contiguous(), scale.contiguous()


def gemm_cases():
    for i, (name, M, N, K, sigma, kw) in enumerate(GEMM_CASES):
        wq, wscale = pack_weight_cpu(weights(N, K, 700 + i, sigma))
        yield name, dict(x=activations(M, K, 600 + i, **kw), wq=wq, wscale=wscale,
                         bias=vector(N, 750 + i, sigma=0.01))


def pack_cases():
    table = (((40, 2048), 1), ((256, 5120), 1), ((1, 16), 0), ((1, 16), 1e-20), ((1, 16), 1e30), ((7, 999), 3))
    for j, (shape, mag) in enumerate(table):
        yield str(j), dict(x=(torch.randn(shape, generator=gen(800 + j)) * mag).to(torch.bfloat16).contiguous())
    patterns = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    yield "all_finite_bf16", dict(x=patterns[torch.isfinite(patterns)].reshape(1, -1).contiguous())


def thor_linear_case():
    w = (torch.randn(1024, 2048, generator=gen(900)) * 0.02).to(torch.bfloat16)
    b = (torch.randn(1024, generator=gen(901)) * 0.01).to(torch.bfloat16)
    return dict(weight=w, bias=b, x=activations(40, 2048, 902))
