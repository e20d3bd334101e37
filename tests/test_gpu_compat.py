"""Drop-in boundary: the same C++ call-site source (tests/cpp/kv_callsite.cu, written the way
the reference's layer loop uses titan::KVCache and cuda::attention_decode) is built once
against the reference's own headers + objects and once against this repo's compat headers +
libtitan_kv.so.  Both binaries run here; their attention outputs must agree."""
import os
import subprocess

import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu

BUILD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp", "_build")


def _run(binary, out, n_tokens, external):
    exe = os.path.join(BUILD, binary)
    assert os.path.exists(exe), f"{exe} missing: run `make -C tests/cpp`"
    res = subprocess.run([exe, out, str(n_tokens), str(int(external))], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"{binary} rc={res.returncode}\n{res.stdout}\n{res.stderr}"
    return np.fromfile(out, dtype=np.float32)


@pytest.mark.parametrize("external", [False, True])
def test_same_call_sites_same_results(tmp_path, external):
    n = 150
    ref = _run("kv_callsite_ref", str(tmp_path / "ref.bin"), n, external)
    ours = _run("kv_callsite_ours", str(tmp_path / "ours.bin"), n, external)
    assert ref.shape == ours.shape == ((n * 2 + 2) * 8 * 64,)
    assert np.abs(ref).max() > 0.1
    # K after RoPE is rounded to fp16 by the paged store; everything else is FP32 on both sides
    assert_close(ours, ref, "compat KVCache + attention_decode vs the reference's own objects")


def test_mla_call_sites_same_results(tmp_path):
    """initialize_external_mla + attention_decode_mla (K rows 192, V rows 128), mode 2 of the program."""
    n = 70
    ref = _run("kv_callsite_ref", str(tmp_path / "ref.bin"), n, 2)
    ours = _run("kv_callsite_ours", str(tmp_path / "ours.bin"), n, 2)
    assert ref.shape == ours.shape == (n * 2 * 8 * 128,)
    assert np.abs(ref).max() > 0.1
    assert_close(ours, ref, "compat MLA KVCache + attention_decode_mla vs the reference's own objects")


def test_storage_types_are_mapped_or_refused_never_substituted(tmp_path):
    """KVCache::initialize(..., DType): FP16 -> fp16 pool, BF16 -> bf16 pool, FP8_E4M3 refused with false (the
    FP8 pool is behind the C ABI); the reference accepts every value because it ignores the argument."""
    exe = os.path.join(BUILD, "kv_callsite_ours")
    res = subprocess.run([exe, str(tmp_path / "x.bin"), "1", "3"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "dtype fp16 1 bf16 1 fp8_e4m3 0" in res.stdout
    assert "FP8-E4M3 pools are behind the C ABI" in res.stderr
