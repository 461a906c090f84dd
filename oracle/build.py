"""Compile the C restatement (``fp8_linear_oracle.c``) into ``oracle/_build/liboracle.so`` with gcc.

``-ffp-contract=off`` is load-bearing: the source spells out which multiply-adds are fused
(``fmaf``) and which are not; the compiler must not contract the others.
"""
from __future__ import annotations

import hashlib
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "fp8_linear_oracle.c"
OUT_DIR = HERE / "_build"
LIBRARY = OUT_DIR / "liboracle.so"
FLAGS = ["-O3", "-march=native", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared",
         "-fvisibility=hidden", "-std=gnu11"]


def build(force: bool = False) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    tag = hashlib.sha256(SOURCE.read_bytes() + " ".join(FLAGS).encode()).hexdigest()[:16]
    stamp = OUT_DIR / "stamp"
    if force or not LIBRARY.exists() or not stamp.exists() or stamp.read_text() != tag:
        cmd = ["gcc", *FLAGS, "-o", str(LIBRARY), str(SOURCE), "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"gcc failed: {' '.join(cmd)}\n{r.stderr}")
        stamp.write_text(tag)
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True))
