"""Record golden vectors of the reference's split-KV attention merge + FP8 row quantiser on a B200.

Runs the unmodified reference's ``_attn_combine`` Triton kernel (instinctflash/kernels/attention.py:109-145,
launched exactly as ``attention()`` launches it at :205-214; the reference is pip-installed,
unchanged, into the git-ignored ``baseline/_ref``) on the seeded partials of
``tests/cases.py::attn_combine_cases`` and writes per case the sha256 of the merged output and of
the e4m3 codes, the per-token scale bits and the first 64 values of the first row.

    python tests/golden/make_golden_gpu_attn.py --out /some/scratch/golden_b200_attn.json

The output is copied to ``tests/golden/golden_b200_attn.json`` and committed.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "tests"))
sys.path.insert(0, str(ROOT / "baseline" / "_ref"))

import cases  # noqa: E402

DEV = "cuda"
E4M3 = torch.float8_e4m3fn


def sha(t):
    t = t.detach().contiguous().cpu()
    if t.dtype == E4M3:
        t = t.view(torch.uint8)
    elif t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    import triton
    from instinctflash.kernels.attention import _attn_combine

    out = dict(device=torch.cuda.get_device_name(0), torch=torch.__version__, cases={})
    for name, c in cases.attn_combine_cases():
        T, HQ, HKV, HD, SP = c["tokens"], c["heads_q"], c["heads_kv"], c["head_dim"], c["splits"]
        po, pm, pl = c["po"].to(DEV), c["pm"].to(DEV), c["pl"].to(DEV)
        o = torch.zeros(1, T, HQ, HD, device=DEV, dtype=c["out_dtype"])
        q8 = torch.zeros(T, HQ * HD, device=DEV, dtype=torch.uint8).view(E4M3)
        qs = torch.zeros(T, device=DEV)
        _attn_combine[(1, T)](po, pm, pl, o, q8, qs, o.stride(0), o.stride(1), o.stride(2), q8.stride(0),
                              T * (HQ // HKV), 1, GROUP=HQ // HKV, HKV=HKV, HEAD_DIM=HD,
                              BLOCK_D=triton.next_power_of_2(HD), SPLITS=SP, WRITE_O=c["write_o"], QUANT=True,
                              num_warps=4)
        torch.cuda.synchronize()
        rec = dict(q_sha=sha(q8), qs_bits=qs.cpu().view(torch.int32).tolist(),
                   q_head=q8[0, :64].cpu().view(torch.uint8).tolist())
        if c["write_o"]:
            rec["o_sha"] = sha(o)
        out["cases"][name] = rec
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps(out))
    print("wrote", args.out, len(out["cases"]), "cases")


if __name__ == "__main__":
    main()
