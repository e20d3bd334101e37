"""The link-level drop-in recipe of INTEGRATION.md, checked on the reference's real callers.

With titan_engine_b200/csrc/compat ahead of the reference's src/ on the include path, the files that
use titan::KVCache and cuda::attention_decode must still compile, `inference/kv_cache.h` must resolve
to the compat header and every other header (core/types.h, compute/dispatch.h, ...) to the reference's
own.  Needs the reference tree (named by BASELINE.json `reference_path`); skipped where it is absent."""
import os
import shutil
import subprocess

import pytest

from oracle import tk_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMPAT = os.path.join(ROOT, "titan_engine_b200", "csrc", "compat")
REF = O.reference_root()
CUDA_INC = next((p for p in ("/usr/local/cuda/include", os.path.join(os.environ.get("CUDA_HOME", "/nonexistent"), "include"))
                 if os.path.exists(os.path.join(p, "cuda_runtime.h"))), None)
CALLERS = ["src/model/dense.cpp", "src/model/moe.cpp", "src/inference/batch.cpp", "src/inference/speculative.cpp",
           "src/inference/engine.cpp"]

needs_reference = pytest.mark.skipif(not REF or not CUDA_INC or not shutil.which("g++"),
                                reason="needs the reference tree, the CUDA headers and g++")


@needs_reference
@pytest.mark.parametrize("caller", CALLERS)
def test_reference_caller_compiles_against_the_compat_header(caller):
    # exactly the include order INTEGRATION.md prescribes: compat first, then the reference's src/
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-I", COMPAT, "-I", os.path.join(REF, "src"), "-I", CUDA_INC,
           os.path.join(REF, caller)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    deps = subprocess.run(cmd[:2] + ["-M"] + cmd[3:], capture_output=True, text=True, check=True).stdout
    deps = {os.path.realpath(p) for p in deps.replace("\\\n", " ").split()[1:]}
    ours = os.path.realpath(os.path.join(COMPAT, "inference", "kv_cache.h"))
    theirs = os.path.realpath(os.path.join(REF, "src", "inference", "kv_cache.h"))
    assert ours in deps and theirs not in deps, "inference/kv_cache.h did not resolve to the compat header"
    assert os.path.realpath(os.path.join(REF, "src", "core", "types.h")) in deps
    inside_compat = {p for p in deps if p.startswith(os.path.realpath(COMPAT) + os.sep)}
    assert inside_compat == {ours}, f"the compat directory shadows more than kv_cache.h: {inside_compat}"


def test_compat_directory_holds_only_the_kv_cache_header_on_the_include_path():
    """Headers for builds outside the reference tree live under compat/standalone, which is NOT on
    the include path of a build inside the reference tree."""
    top = sorted(os.listdir(COMPAT))
    assert top == ["inference", "kv_cache_compat.cu", "standalone"], top
    assert os.listdir(os.path.join(COMPAT, "inference")) == ["kv_cache.h"]
