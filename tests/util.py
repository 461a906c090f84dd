"""Helpers shared by the tests: hashing that matches the golden generators, parity metrics."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

E4M3 = torch.float8_e4m3fn
GOLDEN = Path(__file__).resolve().parent / "golden"

# Parity bar for GEMM outputs against the reference's FP8 path.
REL_FROBENIUS_MAX = 1e-3
ROW_MAX_FRACTION = 2.0 ** -7


def sha(t: torch.Tensor) -> str:
    t = t.detach().contiguous().cpu()
    if t.dtype == E4M3:
        t = t.view(torch.uint8)
    elif t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


def golden(name: str) -> dict:
    return json.loads((GOLDEN / name).read_text())["cases"]


def u8(t):
    return t.detach().cpu().contiguous().view(torch.uint8)


def i32(t):
    return t.detach().cpu().contiguous().view(torch.int32)


def rel_frobenius(got, want) -> float:
    g, w = got.detach().cpu().double(), want.detach().cpu().double()
    return float((g - w).norm() / w.norm().clamp_min(1e-300))


def row_max_fraction(got, want) -> float:
    g, w = got.detach().cpu().double(), want.detach().cpu().double()
    return float(((g - w).abs().amax(1) / w.abs().amax(1).clamp_min(1e-300)).max())


def assert_gemm_parity(got, want, what=""):
    rf, rm = rel_frobenius(got, want), row_max_fraction(got, want)
    assert rf <= REL_FROBENIUS_MAX, f"{what}: relative Frobenius error {rf:.3e} > {REL_FROBENIUS_MAX}"
    assert rm <= ROW_MAX_FRACTION, f"{what}: max|delta| / row absmax {rm:.3e} > 2^-7"


def code_steps(a, b):
    """Distance between two e4m3 code tensors in representable steps (sign-magnitude order)."""
    def order(c):
        c = c.to(torch.int32)
        mag = c & 0x7F
        return torch.where((c & 0x80) != 0, -mag, mag)
    return (order(u8(a)) - order(u8(b))).abs()


def assert_quant_close_to_oracle(q, qs, qo, so, what="", max_scale_ulp=3, max_code_frac=5e-3):
    """The CPU oracle divides in IEEE where the GPU uses div.full.f32 / ex2.approx: scales may
    differ by a few ulp and a code by one step at a rounding boundary, nothing more."""
    ulp = (i32(qs) - i32(so)).abs().max().item()
    assert ulp <= max_scale_ulp, f"{what}: scale differs from the oracle by {ulp} ulp"
    steps = code_steps(q, qo)
    assert steps.max().item() <= 1, f"{what}: a code is {steps.max().item()} steps from the oracle"
    frac = (steps != 0).float().mean().item()
    assert frac <= max_code_frac, f"{what}: {frac:.2%} of codes differ from the oracle"
