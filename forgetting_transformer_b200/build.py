"""Builds the CUDA library in-tree: ``python -m forgetting_transformer_b200.build``.

One ``nvcc`` invocation compiles every kernel file for sm_100a only (SASS, no PTX)
into ``forgetting_transformer_b200/libfox_b200.so``, which exports the C ABI
declared in ``include/fox_b200.h``.  nvcc cross-compiles, so no GPU is needed.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libfox_b200.so")
SOURCES = ["fox_scan.cu", "fox_attn_fwd.cu", "fox_attn_bwd.cu", "fox_attn_bwd_dq.cu", "fox_attn_bwd_kv.cu", "fox_decode.cu", "fox_normgate.cu", "fox_rmsnorm.cu", "fox_shift.cu", "fox_glu.cu", "fox_ce.cu", "fox_noalloc.cu"]
HEADERS = ["fox_common.cuh", "fox_host.h", os.path.join("..", "..", "include", "fox_b200.h")]


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = _sources() + [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [
        nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-o", LIB_PATH,
    ] + (["-Xptxas", "-v"] if verbose else []) + _sources()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
