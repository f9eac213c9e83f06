"""Build libsage_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python sageattention-rdna4_b200/build.py [--force] [--verbose]

The library is plain C-ABI (no libtorch, no Python headers): three translation units linked into
`sageattention/libsage_b200.so` next to the Python package that loads it with ctypes.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "sageattention", "libsage_b200.so")
SOURCES = ["sage_capi.cu", "sage_prologue.cu", "sage_attn_sm100.cu"]
HEADERS = ["sage_common.cuh", "sage_internal.h", os.path.join("..", "..", "include", "sage_b200.h")]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; libsage_b200.so cannot be built")
    return cand


def up_to_date() -> bool:
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return OUT
    cmd = [nvcc_path(), "-std=c++17", "-O3", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-shared", "--threads", "3",
           "-o", OUT] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libsage_b200.so")
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/spill report")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
