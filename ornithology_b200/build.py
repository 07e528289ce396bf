"""Compile the CUDA backend into ornithology_b200/libornith_cuda.so (sm_100a only).

    python -m ornithology_b200.build            # build if sources are newer
    python -m ornithology_b200.build --force

The library is built in-tree so that it travels with the source tree; nothing is
cached elsewhere.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libornith_cuda.so")
INCLUDE = os.path.join(ROOT, "include")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", INCLUDE, "-I", CSRC]
CC_FLAGS = ["-O2", "-std=c11", "-fPIC", "-Wall", "-Wextra", "-pthread", "-I", INCLUDE]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA backend cannot be built")


def sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    c = sorted(f for f in os.listdir(CSRC) if f.endswith(".c"))
    return cu, c


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "ornith_cuda.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    extra = os.environ.get("ORNITH_NVCC_EXTRA", "").split()       # e.g. -DORNITH_SCAN_TRACE for kernel bring-up
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    cu, c = sources()
    logs = {}

    def compile_cu(f):
        o = os.path.join(OBJ, f + ".o")
        r = subprocess.run([nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, f), "-o", o],
                           capture_output=True, text=True)
        logs[f] = r.stderr
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {f}:\n{r.stderr}")
        return o

    def compile_c(f):
        o = os.path.join(OBJ, f + ".o")
        r = subprocess.run(["gcc", *CC_FLAGS, "-c", os.path.join(CSRC, f), "-o", o],
                           capture_output=True, text=True)
        logs[f] = r.stderr
        if r.returncode:
            raise RuntimeError(f"gcc failed on {f}:\n{r.stderr}")
        return o

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_cu, cu)) + list(ex.map(compile_c, c))
    r = subprocess.run([nvcc, "-shared", "-o", LIB, *objs, "-lpthread"], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError(f"link failed:\n{r.stderr}")
    with open(os.path.join(OBJ, "ptxas.log"), "w") as fh:
        for f, t in logs.items():
            fh.write(f"==== {f}\n{t}\n")
    if verbose:
        for f, t in logs.items():
            print(f"==== {f}\n{t}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
