"""Builds libexl3_b200.so (the C-ABI library of sm_100a kernels) in-tree with nvcc.

    python -m trellis_serve_b200.csrc.build [--force] [--verbose]

One object per source; the decode GEMV is compiled once per bit rate (-DEXL3_GEMV_K=2..8) so the seven
instantiation sets build in parallel.  Output: trellis_serve_b200/libexl3_b200.so.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT = os.environ.get("EXL3_B200_BUILD_OUT") or os.path.join(PKG, "libexl3_b200.so")
OBJ = os.environ.get("EXL3_B200_BUILD_OBJ") or os.path.join(HERE, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", 
         "--expt-relaxed-constexpr", "-Xptxas", "-v", *os.environ.get("EXL3_B200_NVCC_FLAGS", "").split()]

PLAIN = ["exl3_api.cu", "exl3_kernels.cu", "exl3_gemv.cu", "exl3_moe.cu", "exl3_moe_tc.cu", "exl3_gemm_tc.cu", "exl3_allreduce.cu", "exl3_step.cu"]
PER_K = [("exl3_gemv_inst.cu", "EXL3_GEMV_K", range(2, 9)), ("exl3_moe_inst.cu", "EXL3_MOE_K", range(2, 9))]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libexl3_b200.so")
    return exe


def _jobs():
    jobs = [(src, os.path.splitext(src)[0] + ".o", []) for src in PLAIN]
    for src, macro, values in PER_K:
        for v in values:
            jobs.append((src, f"{os.path.splitext(src)[0]}_{v}.o", [f"-D{macro}={v}"]))
    return jobs


def _sources_mtime() -> float:
    files = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cu", ".cuh", ".h"))]
    files.append(os.path.join(os.path.dirname(PKG), "include", "exl3_b200.h"))
    return max(os.path.getmtime(f) for f in files)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= _sources_mtime():
        return OUT
    os.makedirs(OBJ, exist_ok=True)
    exe = nvcc()
    logs = []

    def compile_one(job):
        src, obj, defs = job
        cmd = [exe, *ARCH, *FLAGS, *defs, "-c", os.path.join(HERE, src), "-o", os.path.join(OBJ, obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return job, cmd, r

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        results = list(pool.map(compile_one, _jobs()))
    for (src, obj, defs), cmd, r in results:
        logs.append(f"$ {' '.join(cmd)}\n{r.stdout}{r.stderr}")
        if r.returncode != 0:
            sys.stderr.write(logs[-1])
            raise RuntimeError(f"nvcc failed on {src} {defs}")
    with open(os.path.join(OBJ, "ptxas.log"), "w") as f:
        f.write("\n".join(logs))
    if verbose:
        print("\n".join(logs))
    objs = [os.path.join(OBJ, obj) for _, obj, _ in _jobs()]
    cmd = [exe, *ARCH, "-shared", "-o", OUT, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("linking libexl3_b200.so failed")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
