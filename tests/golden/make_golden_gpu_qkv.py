"""Record golden vectors of the reference's QKV consumers on a B200.

Runs the unmodified reference kernels ``qkv_split`` (instinctflash/kernels/rope.py:86-114) and
``wan_qkv`` (instinctflash/kernels/wan.py:85-104), installed with pip into ``baseline/_ref``, on
the seeded inputs of ``tests/cases.py`` and writes per output buffer its sha256, the first 64
elements and every 97th element (as float32 bit patterns).

    python tests/golden/make_golden_gpu_qkv.py --out /some/scratch/golden_b200_qkv.json

The output is copied to ``tests/golden/golden_b200_qkv.json`` and committed.
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
STRIDE = 97


def sha(t: torch.Tensor) -> str:
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


def record(t: torch.Tensor) -> dict:
    flat = t.detach().contiguous().cpu().float().flatten()
    return dict(sha=sha(t), head=flat[:64].view(torch.int32).tolist(), sample=flat[::STRIDE].view(torch.int32).tolist())


def dev(t):
    return None if t is None else t.to(DEV)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    from instinctflash.kernels.rope import qkv_split
    from instinctflash.kernels.wan import wan_qkv

    out = dict(device=torch.cuda.get_device_name(0), torch=torch.__version__, stride=STRIDE, cases={})
    rec = out["cases"]
    for name, c in cases.qkv_split_cases():
        T, HQ, HKV, HD, odt = c["qkv"].shape[0], c["heads_q"], c["heads_kv"], c["head_dim"], c["out_dtype"]
        q = torch.zeros(T, HQ, HD, device=DEV, dtype=odt)
        k = torch.zeros(c["kv_rows"], HKV, HD, device=DEV, dtype=odt)
        v = torch.zeros_like(k)
        base = torch.tensor([c["kv_base"]], device=DEV, dtype=torch.int32) if c["dynamic_base"] else c["kv_base"]
        qkv_split(dev(c["qkv"]), q, k, v, heads_q=HQ, heads_kv=HKV, head_dim=HD, row=dev(c["row"]), col=dev(c["col"]),
                  bias=dev(c["bias"]), inv_freq=dev(c["inv_freq"]), pos=dev(c["pos"]), sections=dev(c["sections"]),
                  q_norm=dev(c["q_norm"]), k_norm=dev(c["k_norm"]), kv_base=base)
        rec[f"qkv_split/{name}"] = dict(q=record(q), k=record(k), v=record(v))
    for name, c in cases.wan_qkv_cases():
        n_rows, D, odt, parts, S = c["raw"].shape[0], c["heads"] * c["head_dim"], c["out_dtype"], c["parts"], c["pool_rows"]
        B = n_rows // c["tokens"]
        q = torch.zeros(n_rows, D, device=DEV, dtype=odt)
        kp = torch.zeros(B, S, D, device=DEV, dtype=odt) if parts >= 2 else None
        vp = torch.zeros(B, S, D, device=DEV, dtype=odt) if parts >= 3 else None
        wan_qkv(dev(c["raw"]), q, heads=c["heads"], head_dim=c["head_dim"], tokens=c["tokens"], k_pool=kp, v_pool=vp,
                slots=dev(c["slots"]), row=dev(c["row"]), col=dev(c["col"]), bias=dev(c["bias"]), q_norm=dev(c["q_norm"]),
                k_norm=dev(c["k_norm"]), pos=dev(c["pos"]), sections=dev(c["sections"]), inv_freq=dev(c["inv_freq"]))
        r = dict(q=record(q))
        if kp is not None:
            r["k"] = record(kp)
        if vp is not None:
            r["v"] = record(vp)
        rec[f"wan_qkv/{name}"] = r
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps(out))
    print("wrote", args.out, len(rec), "cases")


if __name__ == "__main__":
    main()
