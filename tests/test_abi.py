"""The C-ABI library loads and exports every symbol include/et_cuda.h declares (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

import effect_torch_b200 as et
from effect_torch_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "et_cuda.h")).read()
    return sorted(set(re.findall(r"ETC_API\s+[\w\s\*]+?\b(etc_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    assert len(names) >= 50
    for must in ("etc_runtime_create", "etc_qlinear_into", "etc_qlinear_tiled_into", "etc_kv_attention_into", "etc_pool_create",
                 "etc_seq_prefill_match", "etc_decoder_execute_sampled", "etc_rmsnorm_into", "etc_rope_into", "etc_swiglu_into",
                 "etc_argmax_into", "etc_linear_f32_into", "etc_qembedding_into"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"libetcuda.so lacks {name}"


def test_binding_table_matches_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_geometry_helpers_run_without_a_device():
    assert et.encoded_row_bytes(et.Q4_0, 4096) == 128 * 18
    assert et.encoded_row_bytes(et.Q8_0, 4096) == 128 * 34
    assert et.encoded_row_bytes(et.Q4_K, 512) == 288
    with pytest.raises(et.BackendError, match="logical row width 255 is invalid for Q4_K") as e:
        et.encoded_row_bytes(et.Q4_K, 255)
    assert e.value.reason == "compilation-failed"
    # crates/runtime-cpu/src/napi/mod.rs:4922-4953: KV part of the u8-tier state size
    assert et.pool_state_bytes(1, 8, 2, 4, et.KV_U8) == 256
    assert et.pool_state_bytes(1, 8, 2, 4, et.KV_F32) == 512
    out, scratch = C.c_size_t(0), C.c_size_t(0)
    assert _lib.load().etc_qlinear_requirements(et.Q4_K, 2, 2, 512, C.byref(out), C.byref(scratch)) == 0
    assert out.value == 2 * 2 * 4
    assert _lib.load().etc_qlinear_requirements(et.Q4_K, 1, 1, 255, C.byref(out), C.byref(scratch)) == 4  # compilation-failed


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert et.device_count() == 0
    assert et.is_available() is False
    with pytest.raises(et.BackendError) as e:
        et.Runtime(0)
    assert e.value.reason == "backend-unavailable"
    assert "no CPU fallback" in str(e.value)
