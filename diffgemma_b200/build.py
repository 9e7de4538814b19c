"""Builds libdg_attn.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as `python -m diffgemma_b200.build`.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdg_attn.so")


def _nccl_include() -> str:
    try:
        import nvidia.nccl as n  # header only: the library is loaded with dlopen at run time
        inc = os.path.join(list(n.__path__)[0], "include")
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return inc
    except Exception:
        pass
    for cand in ("/usr/include", "/usr/local/cuda/include"):
        if os.path.exists(os.path.join(cand, "nccl.h")):
            return cand
    raise RuntimeError("nccl.h not found")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        [os.path.join(ROOT, "include", "dg_attn.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-ccbin", "/usr/bin/g++", "-Xcompiler", "-fPIC", "-shared",
           "-I", os.path.join(ROOT, "include"), "-I", _nccl_include()]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    # link under a temporary name and rename: a reader never sees a half-written library
    tmp = LIB + ".tmp"
    cmd += sources() + ["-o", tmp, "-ldl"]
    subprocess.check_call(cmd)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
