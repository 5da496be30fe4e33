"""Ahead-of-time build of libminit_b200.so (sm_100a only) with nvcc.

    python minit_b200/csrc/build.py [--force]

(run as a script, or loaded by path: it must work while the library is missing or stale, so it
does not import the minit_b200 package, whose import binds the library's symbols)

Objects go to minit_b200/csrc/_obj/, the library to minit_b200/libminit_b200.so (in-tree, so
it travels with the source tree; both are git-ignored).  A source is recompiled when it or any
header is newer than its object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.dirname(os.path.abspath(__file__))
HERE = os.path.dirname(CSRC)
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libminit_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libminit_b200.so")
    return cand


def _units():
    units = [("dequant.cu", "dequant.o", []), ("api.cu", "api.o", []), ("qgemm_tc.cu", "qgemm_tc.o", []),
             ("qgemm_w8.cu", "qgemm_w8.o", []), ("qgemm_vec.cu", "qgemm_vec.o", []), ("repack.cu", "repack.o", []), ("qgemm_umma.cu", "qgemm_umma.o", []), ("qgemm_mid.cu", "qgemm_mid.o", []), ("qgemm_w8vec.cu", "qgemm_w8vec.o", []), ("decode_ops.cu", "decode_ops.o", []), ("noalloc.cu", "noalloc.o", []), ("nccl_shim.cc", "nccl_shim.o", [])]
    for bits in (4, 8):
        for bf in (0, 1):
            units.append(("qgemm_small_inst.cu", f"qgemm_small_i{bits}_{'bf16' if bf else 'f16'}.o",
                          [f"-DMT_INST_BITS={bits}", f"-DMT_INST_BF16={bf}"]))
    return [u for u in units if os.path.exists(os.path.join(CSRC, u[0]))]


def _headers_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(HERE, "..", "include", "minit_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    hdr = _headers_mtime()
    jobs = []
    for src, obj, defs in _units():
        s, o = os.path.join(CSRC, src), os.path.join(OBJ, obj)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            jobs.append((s, o, defs))

    def run(job):
        s, o, defs = job
        cmd = [nvcc, *NVCC_FLAGS, *defs, "-c", s, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        with open(o + ".log", "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{r.stderr[-4000:]}")
        if verbose:
            print("compiled", os.path.basename(o))
        return o

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            list(ex.map(run, jobs))
    objs = [os.path.join(OBJ, u[1]) for u in _units()]
    if jobs or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr[-4000:])
        if verbose:
            print("linked", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
