"""ctypes declarations for libetcuda.so, one per symbol of include/et_cuda.h.

This is the binding a reference-side addon would write in Rust (`extern "C"` block); tests and the
benchmark call the library only through it. Loading fails loudly when the library is missing:
there is no CPU or PyTorch fallback behind this package.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libetcuda.so")

P = C.c_void_p
I = C.c_int
I64 = C.c_int64
U64 = C.c_uint64
U32 = C.c_uint32
D = C.c_double
SZ = C.c_size_t


class DecoderConfig(C.Structure):
    _fields_ = [
        ("layers", I), ("d_model", I), ("q_heads", I), ("kv_heads", I), ("head_dim", I), ("ffn", I), ("vocab", I),
        ("rms_eps", D), ("rope_theta", D), ("rope_layout", I), ("window", I64), ("batch", I), ("max_tokens", I),
        ("block_size", I), ("kv_dtype", I), ("exact", I),
    ]


class Capabilities(C.Structure):
    _fields_ = [("dtype_mask", U32), ("feature_mask", U32), ("device_ordinal", I), ("sm_count", I), ("compute_major", I),
                ("compute_minor", I), ("device_memory_bytes", U64), ("device_name", C.c_char * 128)]


# name -> (restype, argtypes); restype None means etc_status (int)
SIGNATURES = {
    "etc_last_error_message": (C.c_char_p, []),
    "etc_version": (C.c_char_p, []),
    "etc_device_count": (None, [P]),
    "etc_runtime_create": (None, [I, P]),
    "etc_runtime_destroy": (None, [P]),
    "etc_runtime_stream": (None, [P, P]),
    "etc_runtime_synchronize": (None, [P]),
    "etc_runtime_launch_count": (None, [P, P]),
    "etc_runtime_memory_bytes": (None, [P, P]),
    "etc_runtime_capabilities": (None, [P, P]),
    "etc_alloc": (None, [P, SZ, P]),
    "etc_free": (None, [P, P]),
    "etc_upload": (None, [P, P, P, SZ]),
    "etc_download": (None, [P, P, P, SZ]),
    "etc_encoded_row_bytes": (None, [I, I64, P]),
    "etc_dequantize_into": (None, [P, I, P, I64, I64, P]),
    "etc_quantize_into": (None, [P, I, P, I64, I64, P]),
    "etc_qlinear_requirements": (None, [I, I64, I64, I64, P, P]),
    "etc_qlinear_into": (None, [P, I, P, I64, I64, P, I64, P, P, P]),
    "etc_qweight_create": (None, [P, I, P, P, I, I64, I, I, P]),
    "etc_qweight_destroy": (None, [P]),
    "etc_qweight_shape": (None, [P, P, P, P, P]),
    "etc_qlinear_tiled_scratch_bytes": (None, [P, I64, P]),
    "etc_qlinear_tiled_into": (None, [P, P, P, I64, P, P, I, P, P, SZ]),
    "etc_qlinear_tiled_static_max_bytes": (None, [P]),
    "etc_qlinear_tiled_static_into": (None, [P, P, P, I64, P, P, I, P]),
    "etc_qembedding_into": (None, [P, I, P, I, I64, P, I64, I64, P]),
    "etc_linear_f32_into": (None, [P, P, I64, I64, P, I64, P, P]),
    "etc_rmsnorm_into": (None, [P, P, P, D, I64, I64, P]),
    "etc_rope_into": (None, [P, P, P, I64, D, I, I64, I64, I64, I64, P]),
    "etc_swiglu_into": (None, [P, P, P, I64, P]),
    "etc_add_into": (None, [P, P, P, I64, P]),
    "etc_argmax_into": (None, [P, P, I64, I64, P]),
    "etc_sample_row": (None, [P, P, I64, D, I64, D, U64, U64, P]),
    "etc_sample_rows_into": (None, [P, P, I64, I64, D, I64, D, U64, U64, P, P, P]),
    "etc_pool_create": (None, [P, I, I, I, I, I, I, P]),
    "etc_pool_destroy": (None, [P]),
    "etc_pool_stats": (None, [P, P, P, P]),
    "etc_pool_state_bytes": (None, [I64, I64, I64, I64, I, P]),
    "etc_pool_read_rows": (None, [P, I, I, P, I64, P]),
    "etc_seq_create": (None, [P, P]),
    "etc_seq_release": (None, [P]),
    "etc_seq_destroy": (None, [P]),
    "etc_seq_cursor": (None, [P, P]),
    "etc_seq_prefill_match": (None, [P, P, I64, P]),
    "etc_seq_blocks": (None, [P, P, I64, P, P]),
    "etc_kv_attention_into": (None, [P, P, I, P, I, I, I, P, P, P, I, I, D, I64, I64, P]),
    "etc_kv_append_into": (None, [P, P, I, P, I, I, I, P, P, I, I64]),
    "etc_kv_attention_decode_into": (None, [P, P, I, P, I, I, P, P, P, I, D, I64, I64, P]),
    "etc_seq_commit": (None, [P, P, I, I64]),
    "etc_seq_rollback": (None, [P, I64]),
    "etc_seq_frontier": (None, [P, P]),
    "etc_paged_attention_into": (None, [P, P, I, P, P, I, I, P, I, D, I64, P, P, SZ]),
    "etc_kv_attention_plan": (None, [I, I, I, I, I, I, P, P, P]),
    "etc_decoder_attention_reserve": (None, [P, I, I, P, P]),
    "etc_decoder_create": (None, [P, P, P]),
    "etc_decoder_destroy": (None, [P]),
    "etc_decoder_set_weight": (None, [P, I, I, I, P, I64, I64]),
    "etc_decoder_set_weight_device": (None, [P, I, I, I, P, I64, I64]),
    "etc_decoder_set_max_advance": (None, [P, I]),
    "etc_gguf_open": (None, [C.c_char_p, P, P]),
    "etc_gguf_close": (None, [P]),
    "etc_gguf_summary": (None, [P, P, P, P]),
    "etc_gguf_metadata": (None, [P, I64, P, P, P, P, P, P, P]),
    "etc_gguf_tensor": (None, [P, I64, P, P, P, P, P, P, P]),
    "etc_gguf_find_tensor": (None, [P, C.c_char_p, P]),
    "etc_gguf_read_tensor_into": (None, [P, I64, P, C.c_uint64, P]),
    "etc_gguf_load_tensor_device": (None, [P, P, I64, P, C.c_uint64, P]),
    "etc_tp_unique_id": (None, [P]),
    "etc_decoder_set_tensor_parallel": (None, [P, I, I, P]),
    "etc_decoder_tp_peer_export": (None, [P, P]),
    "etc_decoder_tp_peer_import": (None, [P, P]),
    "etc_decoder_set_head_shard": (None, [P, I64, I64]),
    "etc_decoder_tp_region": (None, [P, P, P]),
    "etc_decoder_tp_peer_attach": (None, [P, P]),
    "etc_decoder_set_wait_limit": (None, [P, I64]),
    "etc_peer_region_bytes": (SZ, [I64, I]),
    "etc_peer_allreduce_into": (None, [P, I, I, P, I64, I, P, P, I64, I, I64]),
    "etc_decoder_finalize": (None, [P]),
    "etc_decoder_execute": (None, [P, P, P, I, P, I, P, P]),
    "etc_decoder_execute_sampled": (None, [P, P, P, I, P, I, P, P]),
    "etc_decoder_generate_greedy": (None, [P, P, P, I, P, I, P, P]),
    "etc_decoder_diagnostics": (None, [P, P, P, P]),
}

_lib = None


def load():
    """Loads libetcuda.so. Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m effect_torch_b200.build` "
            "(the CUDA backend has no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = C.c_int if res is None else res
        fn.argtypes = args
    _lib = lib
    return lib
