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


def test_every_attention_plan_a_step_can_ask_for_fits_the_decoder_reserve():
    """The decoder sets aside split-KV partials once; a captured one-token step plans for the attended pages rounded up
    to 8. Sweep pool capacities and batches (including the geometries where the rounding adds a split: capacities whose
    page count is 1..4 above a multiple of 8 with few lanes) and check that no plan exceeds the reserve."""
    from effect_torch_b200 import DecoderConfig
    for q_heads, kv_heads, head_dim in ((32, 8, 128), (8, 2, 64), (4, 4, 128)):
        for batch in (1, 2, 3, 4, 8, 9, 32, 64):
            for max_tokens in list(range(16, 1025, 16)) + [1600, 2048, 4096, 8192]:
                cfg = DecoderConfig(1, q_heads * head_dim, q_heads, kv_heads, head_dim, 64, 64, 1e-5, 1e4, 0, -1, batch, max_tokens, 16,
                                    et.KV_F16, 0)
                for max_advance in (1, 16):
                    reserve = et.decoder_attention_reserve(cfg, max_advance)
                    assert reserve["max_blocks"] >= max_tokens // 16 + 2
                    for pages in sorted({1, 8, max_tokens // 16, max_tokens // 16 + 1, reserve["max_blocks"]} |
                                        set(range(max(1, max_tokens // 16 - 9), reserve["max_blocks"] + 1))):
                        bucket = (pages + 7) // 8 * 8
                        need = et.attention_plan(batch, q_heads, kv_heads, head_dim, bucket)["partial_bytes"]
                        assert need <= reserve["partial_bytes"], (q_heads, batch, max_tokens, max_advance, pages, need, reserve)
    # a geometry where the rounding matters: 400 tokens (25 pages), one lane, 32 query heads of 128: the 32-page plan has
    # one split more than the 25-page plan and needs 66,560 bytes
    assert et.attention_plan(1, 32, 8, 128, 32)["partial_bytes"] == 66560
    cfg = DecoderConfig(1, 4096, 32, 8, 128, 64, 64, 1e-5, 1e4, 0, -1, 1, 400, 16, et.KV_F16, 0)
    assert et.decoder_attention_reserve(cfg, 1)["partial_bytes"] >= 66560
