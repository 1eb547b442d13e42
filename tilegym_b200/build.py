"""Builds libtilegym_b200.so in-tree with nvcc for sm_100a.

    python -m tilegym_b200.build [--force] [--verbose]

One object per .cu file (compiled in parallel), linked into
tilegym_b200/libtilegym_b200.so with the CUDA runtime linked statically, so the
library has no dependency on torch or on a particular libcudart on the path.
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libtilegym_b200.so")

SOURCES = ["api.cu", "gemm_pertensor.cu", "gemm_pertensor_2cta.cu", "gemm_blockscaled.cu", "gemm_blockscaled_wide.cu", "gemm_blockscaled_smallm.cu", "gemm_smallm.cu", "quant.cu", "group_quant.cu", "no_alloc.cu", "selftest.cu", "moe.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(PKG_DIR, "..", "include", "tilegym_b200.h"))
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        if force or not _newer(o, [s] + headers):
            extra = os.environ.get("TILEGYM_B200_NVCC_EXTRA", "").split()  # e.g. -DTG_TRACE for phase stamps
            cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append((src, cmd))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            futs = {ex.submit(subprocess.run, cmd, capture_output=True, text=True): src for src, cmd in jobs}
            for f in cf.as_completed(futs):
                r = f.result()
                if verbose or r.returncode != 0:
                    sys.stderr.write(f"--- {futs[f]}\n{r.stdout}{r.stderr}")
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {futs[f]}")
    objs = [os.path.join(OBJ_DIR, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or not _newer(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs + ["-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
