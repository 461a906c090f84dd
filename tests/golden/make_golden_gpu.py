"""Record golden vectors of the reference's OWN FP8 path on a B200.

Runs the unmodified InstinctFlash reference (installed with pip, unchanged, into the git-ignored
``baseline/_ref``) on the seeded inputs of ``tests/cases.py`` and writes ``golden_b200.json``:
per case the sha256 of every output buffer, the full per-row scale vectors (as int32 bit
patterns) and the first 64 elements of the first row of each buffer.  The Triton kernels of ``instinctflash.kernels`` have no
capability gate and run on sm_100 as they are; the per-tensor packer does have one
(instinctflash/runtime/fp8_pack.py:48-50), so ``torch.cuda.get_device_capability`` is patched
to (9, 0) around it, the way the reference's own tests do (tests/test_sm89_fp8.py:52).

    python tests/golden/make_golden_gpu.py --out /some/scratch/golden_b200.json

The output is copied to ``tests/golden/golden_b200.json`` and committed.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path
from unittest.mock import patch

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "tests"))
sys.path.insert(0, str(ROOT / "baseline" / "_ref"))

import cases  # noqa: E402

DEV = "cuda"
E4M3 = torch.float8_e4m3fn


def sha(t: torch.Tensor) -> str:
    t = t.detach().contiguous().cpu()
    if t.dtype == E4M3:
        t = t.view(torch.uint8)
    elif t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


HEAD = 64  # elements of the first row kept verbatim next to each hash


def bits32(t: torch.Tensor):
    return t.detach().contiguous().cpu().view(torch.int32).tolist()


def head32(t: torch.Tensor):
    return t[0, :HEAD].detach().contiguous().cpu().view(torch.int32).tolist()


def head16(t: torch.Tensor):
    return t[0, :HEAD].detach().contiguous().cpu().view(torch.int16).tolist()


def codes(t: torch.Tensor):
    return t[0, :HEAD].detach().contiguous().cpu().view(torch.uint8).tolist()


def quant_record(q, qs):
    return dict(q_sha=sha(q), qs_sha=sha(qs), qs_bits=bits32(qs), q_head=codes(q))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()

    from instinctflash.kernels.activation import GELU_TANH, SILU, gated_act_quant
    from instinctflash.kernels.fp8 import Fp8Weight, gemm
    from instinctflash.kernels.norm import dequant_rows, residual_norm_quant, row_quant

    out = dict(device=torch.cuda.get_device_name(0), torch=torch.__version__, cases={})
    rec = out["cases"]

    def dev(t):
        return None if t is None else t.to(DEV)

    # ---- row_quant, plain (bf16 / fp16 / fp32 inputs) -----------------------------------
    for name, c in cases.row_quant_cases():
        x = dev(c["x"])
        q = torch.empty(x.shape, device=DEV, dtype=E4M3)
        qs = torch.empty(x.shape[0], device=DEV, dtype=torch.float32)
        row_quant(x, q, qs)
        rec[f"row_quant/{name}"] = quant_record(q, qs)

    # ---- row_quant with the consumer prologue (raw accumulator in) ---------------------
    for name, c in cases.prologue_cases():
        x = dev(c["x"])
        q = torch.empty(x.shape, device=DEV, dtype=E4M3)
        qs = torch.empty(x.shape[0], device=DEV)
        row_quant(x, q, qs, row=dev(c["row"]), col=dev(c["col"]), bias=dev(c["bias"]), gelu=c["gelu"])
        rec[f"row_quant_prologue/{name}"] = quant_record(q, qs)

    # ---- gated_act_quant ---------------------------------------------------------------
    for name, c in cases.gated_cases():
        gu = dev(c["gu"])
        M, F = gu.shape[0], gu.shape[1] // 2
        q = torch.empty(M, F, device=DEV, dtype=E4M3)
        qs = torch.empty(M, device=DEV)
        gated_act_quant(gu, q, qs, row=dev(c["row"]), col=dev(c["col"]), act=c["act"])
        rec[f"gated_act_quant/{name}"] = quant_record(q, qs)

    # ---- dequant_rows ------------------------------------------------------------------
    for name, c in cases.dequant_cases():
        x = dev(c["x"])
        y = torch.empty(x.shape, device=DEV, dtype=c["out_dtype"])
        dequant_rows(x, y, row=dev(c["row"]), col=dev(c["col"]), bias=dev(c["bias"]))
        r = dict(y_sha=sha(y))
        r["y_head"] = head32(y) if c["out_dtype"] == torch.float32 else head16(y)
        y2 = torch.empty_like(y)
        dequant_rows(x, y2, row=dev(c["row"]), col=dev(c["col"]))
        r["y_nobias_sha"] = sha(y2)
        rec[f"dequant_rows/{name}"] = r

    # ---- residual_norm_quant -----------------------------------------------------------
    for name, c in cases.resnorm_cases():
        res = dev(c["res"]).clone()
        M, D = res.shape
        q = torch.empty(M, D, device=DEV, dtype=E4M3)
        qs = torch.empty(M, device=DEV)
        residual_norm_quant(res, delta=dev(c["delta"]), delta_row=dev(c["delta_row"]), delta_col=dev(c["delta_col"]),
                            bias=dev(c["bias"]), gate=dev(c["gate"]), layernorm=c["layernorm"], weight=dev(c["weight"]),
                            beta=dev(c["beta"]), mod_scale=dev(c["mod_scale"]), mod_shift=dev(c["mod_shift"]),
                            mod_index=dev(c["mod_index"]), q=q, q_scale=qs)
        r = quant_record(q, qs)
        r["res_sha"] = sha(res)
        r["res_head"] = head32(res) if res.dtype == torch.float32 else head16(res)
        r["deq_head"] = (q[0, :HEAD].float() * qs[0]).cpu().tolist()
        rec[f"residual_norm_quant/{name}"] = r

    # ---- gemm (torch._scaled_mm / cuBLASLt on this GPU) --------------------------------
    for name, c in cases.gemm_cases():
        x = dev(c["x"])
        M, K = x.shape
        a = torch.empty(M, K, device=DEV, dtype=E4M3)
        s = torch.empty(M, device=DEV)
        row_quant(x, a, s)
        W = Fp8Weight(dev(c["wq"]), dev(c["wscale"]), None)
        raw = torch.empty(M, W.w.shape[0], device=DEV, dtype=torch.bfloat16)
        gemm(a, W, raw)
        y = torch.empty(M, W.w.shape[0], device=DEV, dtype=torch.bfloat16)
        dequant_rows(raw, y, row=s, col=W.scale, bias=dev(c["bias"]))
        rec[f"gemm/{name}"] = dict(a=quant_record(a, s), w_sha=sha(c["wq"]), raw_sha=sha(raw),
                                   raw_head=head16(raw), y_sha=sha(y), y_head=head16(y))

    # ---- per-tensor recipe (fp8_pack.py, torch_fp8_linear.py) ---------------------------
    with patch.object(torch.cuda, "get_device_capability", return_value=(9, 0)):
        from instinctflash.runtime.fp8_pack import dynamic_pack_bf16_e4m3
        from instinctflash.runtime.torch_fp8_linear import ThorFP8Linear
        for name, c in cases.pack_cases():
            packed, scale = dynamic_pack_bf16_e4m3(dev(c["x"]))
            rec[f"dynamic_pack/{name}"] = dict(q_sha=sha(packed), scale_bits=bits32(scale), q_head=codes(packed))
        c = cases.thor_linear_case()
        lin = torch.nn.Linear(2048, 1024, bias=True, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(c["weight"])
            lin.bias.copy_(c["bias"])
        lin = lin.to(DEV)
        mod = ThorFP8Linear(lin, device=DEV)
        y = mod(dev(c["x"]))
        rec["thor_fp8_linear/40x1024x2048"] = dict(weight_sha=sha(mod.weight_fp8),
                                                   weight_scale_bits=bits32(mod.weight_scale),
                                                   y_sha=sha(y), y_head=head16(y))

    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps(out))
    print("wrote", args.out, len(rec), "cases")


if __name__ == "__main__":
    main()
