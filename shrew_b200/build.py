"""Builds libshrewq.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m shrew_b200.build [--force] [--verbose] [--trace]

nvcc cross-compiles without a GPU.  The shared object lands beside this file so that it
travels with the source tree; nothing is written outside the package directory.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libshrewq.so")
SOURCES = ["api.cu", "quantize.cu", "quantize_batch.cu", "quantize_modes.cu", "gemv.cu", "gemv_mma.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "gemm_tcgen05_2cta.cu", "exchange.cu"]
HEADERS = sorted(os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith(".cuh")) + [os.path.join(HERE, "..", "include", "shrewq.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """trace=True builds libshrewq_trace.so: the same library with -DSHREWQ_TRACE, whose
    tcgen05 kernel stamps clock64() per pipeline role and stage."""
    if trace:
        return _build(os.path.join(CSRC, "build_trace"), os.path.join(HERE, "libshrewq_trace.so"),
                      FLAGS + ["-DSHREWQ_TRACE"], force, verbose)
    return _build(os.path.join(CSRC, "build"), LIB, FLAGS, force, verbose)


def _build(objdir: str, lib: str, flags: list[str], force: bool, verbose: bool) -> str:
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + HEADERS):
            cmd = [NVCC, *flags, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1) or 1) as ex:
        list(ex.map(run, jobs))
    objs = [os.path.join(objdir, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(lib, objs):
        run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib, *objs, "-cudart", "static"])
    return lib


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
