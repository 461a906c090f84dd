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


def rope_inv_freq(head_dim, theta=10000.0):
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
    return (1.0 / (theta ** exponent)).float()


def qkv_split_cases():
    """(name, kwargs) for the split of a fused QKV accumulator; flag sets follow the reference's
    call sites (instinctflash/engines/pi05/engine.py:200-201,231-233, vla4/engine.py:124-126,
    vla2/engine.py:158-160) plus ragged and float32 variants."""
    table = [  # name, T, HQ, HKV, HD, xdt, odt, row, bias, norm, rope, sections, kv_rows, kv_base, dynamic
        ("pi05_prefix", 96, 8, 1, 256, torch.bfloat16, torch.float16, True, False, False, True, 0, 128, 0, False),
        ("pi05_expert", 50, 8, 1, 256, torch.bfloat16, torch.float16, True, False, False, True, 0, 128, 37, True),
        ("vla4_bias", 64, 4, 2, 128, torch.bfloat16, torch.float16, True, True, False, True, 0, 64, 0, False),
        ("vla2_mrope_norm", 33, 6, 2, 128, torch.bfloat16, torch.bfloat16, True, False, True, True, 3, 48, 9, True),
        ("ragged_plain", 5, 3, 1, 80, torch.bfloat16, torch.bfloat16, False, True, False, False, 0, 8, 2, False),
        ("f32_norm", 7, 2, 2, 64, torch.float32, torch.float32, True, True, True, True, 2, 16, 4, False),
    ]
    for j, (name, T, HQ, HKV, HD, xdt, odt, use_row, use_bias, norm, rope, nsec, kv_rows, kv_base, dyn) in enumerate(table):
        width = (HQ + 2 * HKV) * HD
        S = max(nsec, 1)
        pos = None
        if rope:
            g = gen(760 + j)
            pos = (torch.rand(T, S, generator=g) * 800.0).floor()
        yield name, dict(
            qkv=raw_like(T, width, 700 + j).to(xdt), heads_q=HQ, heads_kv=HKV, head_dim=HD, out_dtype=odt,
            row=vector(T, 710 + j, lo=0.001, hi=0.02) if use_row else None,
            col=vector(width, 720 + j, lo=0.05, hi=0.5), bias=vector(width, 730 + j, sigma=0.3) if use_bias else None,
            q_norm=vector(HD, 740 + j, lo=0.5, hi=1.5) if norm else None,
            k_norm=vector(HD, 750 + j, lo=0.5, hi=1.5) if norm else None,
            inv_freq=rope_inv_freq(HD) if rope else None, pos=pos,
            sections=(torch.arange(HD // 2, dtype=torch.int32) % nsec) if nsec else None,
            kv_rows=kv_rows, kv_base=kv_base, dynamic_base=dyn)


def wan_qkv_cases():
    """Wan projection consumer; flag sets of instinctflash/engines/wan_va/engine.py:183-184 (text
    K from a [K | V] accumulator), :215-217 (self-attention Q/K/V with pooled K/V) and :226-227
    (cross-attention Q), plus a ragged width and the 14B width."""
    table = [  # name, B, T, H, HD, parts, raw_parts, odt, row, col, bias, qn, kn, rope, slots, S
        ("self_attn", 2, 40, 24, 128, 3, 3, torch.float16, True, True, True, True, True, True, True, 64),
        ("cross_q", 2, 24, 24, 128, 1, 1, torch.float16, True, True, True, True, False, False, False, 0),
        ("text_k", 2, 16, 24, 128, 1, 2, torch.float16, True, True, True, True, False, False, False, 0),
        ("ragged_kv", 1, 9, 5, 4, 2, 2, torch.bfloat16, False, False, True, False, True, True, False, 9),
        ("wide_14b", 1, 16, 40, 128, 3, 3, torch.bfloat16, True, True, True, True, True, True, False, 16),
    ]
    for j, (name, B, T, H, HD, parts, raw_parts, odt, use_row, use_col, use_bias, qn, kn, rope, use_slots, S) in enumerate(table):
        D = H * HD
        rows_n = B * T
        g = gen(860 + j)
        yield name, dict(
            raw=raw_like(rows_n, raw_parts * D, 800 + j), heads=H, head_dim=HD, tokens=T, parts=parts, out_dtype=odt,
            row=vector(rows_n, 810 + j, lo=0.001, hi=0.02) if use_row else None,
            col=vector(parts * D, 820 + j, lo=0.05, hi=0.5) if use_col else None,
            bias=vector(parts * D, 830 + j, sigma=0.3) if use_bias else None,
            q_norm=vector(D, 840 + j, lo=0.5, hi=1.5) if qn else None,
            k_norm=vector(D, 850 + j, lo=0.5, hi=1.5) if kn else None,
            inv_freq=rope_inv_freq(HD) if rope else None,
            pos=(torch.rand(T, 3, generator=g) * 60.0).floor() if rope else None,
            sections=(torch.arange(HD // 2, dtype=torch.int32) % 3) if rope else None,
            slots=torch.randperm(S, generator=g)[:T].to(torch.int32) if use_slots else None, pool_rows=S)


def attn_combine_cases():
    """Split-KV attention partials as the reference's attention kernel leaves them: unnormalised
    output vectors, running maxima (base-2 exponent domain) and running sums per split.  Geometries
    of the engines' call sites: pi05 / VLA grouped-query heads (8 q heads on 1 kv head, width 256),
    LingBot-VLA (width 128, 2 kv heads), Wan (24 heads of 128, no grouping), SigLIP-like width 72."""
    table = [  # name, tokens, hq, hkv, head_dim, splits, out dtype, write_o
        ("pi05_expert", 50, 8, 1, 256, 4, torch.float16, True),
        ("vla4", 51, 4, 2, 128, 3, torch.float16, False),
        ("wan", 33, 24, 24, 128, 2, torch.bfloat16, True),
        ("width72", 9, 16, 16, 72, 2, torch.float16, True),
        ("one_split", 5, 8, 2, 64, 1, torch.float32, True),
    ]
    for j, (name, T, HQ, HKV, HD, SP, odt, write_o) in enumerate(table):
        g = gen(950 + j)
        rows = T * (HQ // HKV)
        width = 1 << max(0, (HD - 1).bit_length())
        pm = torch.randn(SP, 1, HKV, rows, generator=g) * 4.0
        pl = torch.rand(SP, 1, HKV, rows, generator=g) * 30.0 + 1.0
        po = torch.randn(SP, 1, HKV, rows, width, generator=g) * pl[..., None] * 0.3
        yield name, dict(po=po.contiguous(), pm=pm.contiguous(), pl=pl.contiguous(), tokens=T, heads_q=HQ, heads_kv=HKV,
                         head_dim=HD, splits=SP, out_dtype=odt, write_o=write_o)


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
