"""Builds libtitan_kv.so (CUDA kernels + C ABI) for sm_100a, in-tree, with nvcc.

nvcc cross-compiles without a GPU.  The library is what the package loads; there is
no other compute path.  Every source is compiled to an object of its own (in parallel,
only when it or a header changed) and the objects are linked into the shared library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libtitan_kv.so")
SOURCES = ["titan_kv.cu", "append.cu", "decode_simt.cu", "decode_mma.cu", "decode_mma_mla.cu", "prefill_mma.cu", "prefill_tc.cu",
           "decode_static.cu", "peer_exchange.cu", "rope_append.cu", "kv_manager.cpp", "kv_scheduler.cpp",
           "sched_abi.cpp", "compat/kv_cache_compat.cu"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def headers() -> list[str]:
    deps = [os.path.join(HERE, "..", "include", "titan_kv.h")]
    for root, _, files in os.walk(CSRC):
        deps += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh"))]
    return deps


def obj_path(src: str) -> str:
    return os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in sources() + headers() if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = nvcc_path()
    inc = ["-I", os.path.join(HERE, "..", "include"), "-I", CSRC, "-I", os.path.join(CSRC, "compat"),
           "-I", os.path.join(CSRC, "compat", "standalone")]
    hdr_time = max(os.path.getmtime(h) for h in headers())

    def compile_one(src: str) -> tuple[str, int, str]:
        obj = obj_path(src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), hdr_time):
            return obj, 0, ""
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), *inc, "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return obj, res.returncode, res.stdout + res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    for _, rc, log in results:
        if rc != 0 or verbose:
            sys.stderr.write(log)
    if any(rc != 0 for _, rc, _ in results):
        raise RuntimeError("nvcc failed building libtitan_kv.so")
    res = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB,
                          *[o for o, _, _ in results]], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed linking libtitan_kv.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
