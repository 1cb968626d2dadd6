"""Builds libmegafold_b200.so in-tree with nvcc for sm_100a.

    python -m megafold_b200.build [--force] [--verbose]

The library is plain CUDA C++ behind a C ABI (include/megafold_b200.h); it links the static CUDA
runtime only, so it loads on hosts without a GPU driver (entry points then fail with MF_ERR_CUDA).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
# MF_TRACE=1 in the environment builds the phase-trace variant (-DMF_TRACE, see csrc/evo_tc_common.cuh) next to the
# regular library; megafold_b200._lib loads it when MF_TRACE=1 is set there too.
TRACE = os.environ.get("MF_TRACE") == "1"
LIB = os.path.join(PKG, "libmegafold_b200_trace.so" if TRACE else "libmegafold_b200.so")
OBJ_DIR = os.path.join(PKG, "build_trace" if TRACE else "build")

SOURCES = ["api.cu", "evo_simt.cu", "evo_tc.cu", "evo_tc_fwd.cu", "evo_fwd_ws.cu", "evo_bwd_ws.cu", "lnl_ops.cu", "lnl_tc.cu", "transition_tc.cu", "gemm_tc.cu", "transition_bwd_tc.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the megafold_b200 library cannot be built")


def _deps(src: str):
    yield os.path.join(CSRC, src)
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".h")):
            yield os.path.join(CSRC, f)
    yield os.path.join(ROOT, "include", "megafold_b200.h")
    yield os.path.abspath(__file__)


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in SOURCES:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        if force or _stale(obj, _deps(src)):
            cmd = [nvcc, *NVCC_FLAGS, *(["-DMF_TRACE"] if TRACE else []), "-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + p.stdout + p.stderr)
        return p.stdout + p.stderr

    with ThreadPoolExecutor(max_workers=4) as ex:
        for out in ex.map(run, jobs):
            if verbose and out.strip():
                print(out)
    objs = [os.path.join(OBJ_DIR, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC", "-cudart", "static", "-ldl"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
