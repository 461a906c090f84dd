"""Record golden vectors of the reference's CPU-runnable pieces (run in the build container).

Imports the unmodified reference from its source tree and runs, on the seeded inputs of
``tests/cases.py``: ``quantize_weight`` (pure torch; instinctflash/kernels/fp8.py:30-37) and
``gemm`` (``torch._scaled_mm`` has a CPU path for unit scales; fp8.py:50-53).  The Triton
kernels cannot run without a GPU; their vectors are recorded on a B200 by ``make_golden_gpu.py``.

    python tests/golden/make_golden_cpu.py /path/to/InstinctFlash

writes ``tests/golden/golden_cpu.json``.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden_cpu.py /path/to/InstinctFlash")
sys.path.insert(0, sys.argv[1])

import cases  # noqa: E402
from instinctflash.kernels.fp8 import Fp8Weight, gemm, quantize_weight  # noqa: E402

E4M3 = torch.float8_e4m3fn


def sha(t):
    t = t.detach().contiguous().cpu()
    if t.dtype == E4M3:
        t = t.view(torch.uint8)
    elif t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


def main():
    rec = {}
    for i, (N, K, sigma) in enumerate([(4096, 1024, 0.02), (2560, 2048, 0.02), (1536, 1024, 0.02), (48, 16, 1.0)]):
        w = cases.weights(N, K, 1000 + i, sigma)
        b = cases.vector(N, 1100 + i, sigma=0.01).to(torch.bfloat16)
        fw = quantize_weight(w, b)
        rec[f"quantize_weight/{i}"] = dict(N=N, K=K, sigma=sigma, w_sha=sha(fw.w), scale_sha=sha(fw.scale),
                                           scale_head=fw.scale[:64].view(torch.int32).tolist(), bias_sha=sha(fw.bias))
    # zero rows exercise the 1e-12 floor
    w = cases.weights(32, 64, 1010, 0.02)
    w[3] = 0
    fw = quantize_weight(w)
    rec["quantize_weight/zero_row"] = dict(w_sha=sha(fw.w), scale_bits=fw.scale.view(torch.int32).tolist())
    # raw-accumulator GEMM on the CPU (mkldnn), inputs = IEEE-quantised activations and weights
    for name, c in list(cases.gemm_cases())[:1] + [t for t in cases.gemm_cases() if t[0] in ("c3_qkv", "tiny", "tail_k", "tail_n")]:
        x = c["x"].float()
        amax = x.abs().amax(1).clamp_min(1e-8)
        a = (x * (448.0 / amax)[:, None]).to(E4M3)
        W = Fp8Weight(c["wq"], c["wscale"], None)
        raw = torch.empty(a.shape[0], W.w.shape[0], dtype=torch.bfloat16)
        gemm(a, W, raw)
        rec[f"gemm_cpu/{name}"] = dict(a_sha=sha(a), raw_sha=sha(raw), raw_head=raw[0, :64].view(torch.int16).tolist(),
                                       row_sums=raw.double().sum(1).tolist(), row_abs_sums=raw.double().abs().sum(1).tolist())
    (HERE / "golden_cpu.json").write_text(json.dumps(dict(torch=torch.__version__, cases=rec)))
    print("wrote", HERE / "golden_cpu.json", len(rec), "cases")


if __name__ == "__main__":
    main()
