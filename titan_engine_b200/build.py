"""Builds libtitan_kv.so (CUDA kernels + C ABI) for sm_100a, in-tree, with nvcc.

nvcc cross-compiles without a GPU.  The library is what the package loads; there is
no other compute path.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtitan_kv.so")
SOURCES = ["titan_kv.cu", "append.cu", "decode_simt.cu", "decode_mma.cu", "decode_mma_mla.cu", "decode_static.cu", "peer_exchange.cu", "rope_append.cu",
           "kv_manager.cpp", "kv_scheduler.cpp", "sched_abi.cpp", "compat/kv_cache_compat.cu"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-shared"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    compat = os.path.join(CSRC, "compat")
    if os.path.isdir(compat):
        deps += [os.path.join(compat, f) for f in os.listdir(compat)]
    deps.append(os.path.join(HERE, "..", "include", "titan_kv.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS, "-I", os.path.join(HERE, "..", "include"), "-I", CSRC,
           "-I", os.path.join(CSRC, "compat"),
           "-o", LIB, *sources()]
    cmd += os.environ.get("TK_NVCC_DEFS", "").split()     # experiments: e.g. -DTK_MMA_STAGES=2
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libtitan_kv.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
