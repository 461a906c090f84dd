"""Build ``libiflb200.so`` (sm_100a) in-tree with nvcc.

Run as ``python -m instinctflash_b200.build`` or call :func:`build`.  nvcc cross-compiles
without a GPU.  Objects are cached by a hash of the sources and flags under ``csrc/_obj``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIBRARY = PKG / "libiflb200.so"
# (source, extra defines, object stem): row_ops.cu is compiled as three translation units in parallel
SOURCES = (("gemm_fp8_sm100.cu", (), "gemm_fp8_sm100"),
           ("stack_persistent.cu", (), "stack_persistent"),
           ("qkv_ops.cu", (), "qkv_ops"),
           ("attn_ops.cu", (), "attn_ops"),
           ("xgpu_ops.cu", (), "xgpu_ops"),
           ("row_ops.cu", ("-DIFLB200_ROW_PART=0",), "row_ops_quant"),
           ("row_ops.cu", ("-DIFLB200_ROW_PART=1",), "row_ops_gated_pack"),
           ("row_ops.cu", ("-DIFLB200_ROW_PART=2",), "row_ops_resnorm"))
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
)


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libiflb200.so")
    return found


def _digest(paths) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def build(force: bool = False, verbose: bool = False) -> Path:
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    obj_dir = CSRC / "_obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objects, jobs = [], []
    for name, defines, stem in SOURCES:
        src = CSRC / name
        tag = _digest([src] + headers)
        obj = obj_dir / f"{stem}.{tag}.o"
        objects.append(obj)
        if force or not obj.exists():
            for old in obj_dir.glob(f"{stem}.*.o"):
                old.unlink()
            cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
            list(pool.map(run, jobs))
    stamp = obj_dir / "link.stamp"
    want = " ".join(o.name for o in objects)
    if jobs or not LIBRARY.exists() or not stamp.exists() or stamp.read_text() != want:
        run([nvcc, "-shared", "-Xcompiler", "-fPIC", "-o", str(LIBRARY), *map(str, objects)])
        stamp.write_text(want)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
