//! Raw bindings to `libetcuda.so`, the CUDA backend's C ABI (`include/et_cuda.h`): one declaration per exported symbol, in
//! header order, with the header's parameter names. Pointers whose name starts with `d_` are device addresses, `h_`
//! host addresses; `*const c_int` cancellation flags are read by the library with volatile loads while a call runs.
//! Every function returning [`EtcStatus`] leaves its message in a thread-local string read by
//! [`etc_last_error_message`]; the safe layer in `lib.rs` turns a non-zero status into `BackendError`.
//!
//! This crate plays for CUDA the part `crates/runtime-cpu` plays for the host: `crates/runtime-cpu/src/lib.rs` exposes
//! the kernels to Rust callers, `crates/runtime-cpu/src/napi/mod.rs` the addon classes to JavaScript.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_void};

/// `etc_status`: 0 is success; the other values name the `BackendError` reason (packages/core/src/Runtime.ts:129-143).
pub type EtcStatus = c_int;
pub const ETC_OK: EtcStatus = 0;
pub const ETC_UNAVAILABLE: EtcStatus = 1;
pub const ETC_UNSUPPORTED: EtcStatus = 2;
pub const ETC_INVALID_HANDLE: EtcStatus = 3;
pub const ETC_COMPILATION: EtcStatus = 4;
pub const ETC_EXECUTION: EtcStatus = 5;
pub const ETC_TRANSFER: EtcStatus = 6;
pub const ETC_CANCELLED: EtcStatus = 7;
pub const ETC_CLOSED: EtcStatus = 8;
pub const ETC_INVALID_ARGUMENT: EtcStatus = 9;

/// `etc_codec`: GGML type codes (crates/runtime/src/gguf.rs:201-226 plus the 32-value block codecs).
pub const ETC_CODEC_F32: c_int = 0;
pub const ETC_CODEC_Q4_0: c_int = 2;
pub const ETC_CODEC_Q8_0: c_int = 8;
pub const ETC_CODEC_Q2_K: c_int = 10;
pub const ETC_CODEC_Q3_K: c_int = 11;
pub const ETC_CODEC_Q4_K: c_int = 12;
pub const ETC_CODEC_Q5_K: c_int = 13;
pub const ETC_CODEC_Q6_K: c_int = 14;

/// `etc_kv_dtype` (crates/runtime-cpu/src/pool.rs:20-25).
pub const ETC_KV_F32: c_int = 0;
pub const ETC_KV_F16: c_int = 1;
pub const ETC_KV_BF16: c_int = 2;
pub const ETC_KV_U8: c_int = 3;

/// `etc_rope_layout`, `etc_index_dtype`, `etc_epilogue`.
pub const ETC_ROPE_HALF_SPLIT: c_int = 0;
pub const ETC_ROPE_INTERLEAVED_PAIRS: c_int = 1;
pub const ETC_INDEX_U32: c_int = 0;
pub const ETC_INDEX_I64: c_int = 1;
pub const ETC_EPILOGUE_NONE: c_int = 0;
pub const ETC_EPILOGUE_RESIDUAL: c_int = 1;
pub const ETC_EPILOGUE_SWIGLU: c_int = 2;

/// `etc_weight_slot`.
pub const ETC_W_TOK_EMBD: c_int = 0;
pub const ETC_W_ATTN_NORM: c_int = 1;
pub const ETC_W_Q: c_int = 2;
pub const ETC_W_K: c_int = 3;
pub const ETC_W_V: c_int = 4;
pub const ETC_W_O: c_int = 5;
pub const ETC_W_FFN_NORM: c_int = 6;
pub const ETC_W_GATE: c_int = 7;
pub const ETC_W_UP: c_int = 8;
pub const ETC_W_DOWN: c_int = 9;
pub const ETC_W_OUT_NORM: c_int = 10;
pub const ETC_W_HEAD: c_int = 11;

pub const ETC_NO_WINDOW: i64 = -1;

macro_rules! opaque {
    ($($name:ident),*) => { $( #[repr(C)] pub struct $name { _private: [u8; 0] } )* };
}
opaque!(EtcRuntime, EtcPool, EtcSeq, EtcQweight, EtcDecoder, EtcGguf);

/// `etc_capabilities`.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct EtcCapabilities {
    pub dtype_mask: u32,
    pub feature_mask: u32,
    pub device_ordinal: c_int,
    pub sm_count: c_int,
    pub compute_major: c_int,
    pub compute_minor: c_int,
    pub device_memory_bytes: u64,
    pub device_name: [c_char; 128],
}

/// `etc_decoder_config`.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct EtcDecoderConfig {
    pub layers: c_int,
    pub d_model: c_int,
    pub q_heads: c_int,
    pub kv_heads: c_int,
    pub head_dim: c_int,
    pub ffn: c_int,
    pub vocab: c_int,
    pub rms_eps: f64,
    pub rope_theta: f64,
    pub rope_layout: c_int,
    pub window: i64,
    pub batch: c_int,
    pub max_tokens: c_int,
    pub block_size: c_int,
    pub kv_dtype: c_int,
    pub exact: c_int,
}

/// `etc_lane`: one sequence of a step as the attention kernels read it from device memory.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct EtcLane {
    pub cursor: c_int,
    pub advance: c_int,
    pub start: c_int,
    pub table_offset: c_int,
}

#[link(name = "etcuda")]
extern "C" {
    pub fn etc_last_error_message() -> *const c_char;
    pub fn etc_version() -> *const c_char;
    pub fn etc_device_count(out_count: *mut c_int) -> EtcStatus;
    pub fn etc_runtime_create(device_ordinal: c_int, out: *mut *mut EtcRuntime) -> EtcStatus;
    pub fn etc_runtime_destroy(rt: *mut EtcRuntime) -> EtcStatus;
    pub fn etc_runtime_stream(rt: *mut EtcRuntime, out_stream: *mut *mut c_void) -> EtcStatus;
    pub fn etc_runtime_synchronize(rt: *mut EtcRuntime) -> EtcStatus;
    pub fn etc_runtime_launch_count(rt: *mut EtcRuntime, out: *mut u64) -> EtcStatus;
    pub fn etc_runtime_memory_bytes(rt: *mut EtcRuntime, out: *mut u64) -> EtcStatus;
    pub fn etc_runtime_capabilities(rt: *mut EtcRuntime, out: *mut EtcCapabilities) -> EtcStatus;
    pub fn etc_alloc(rt: *mut EtcRuntime, bytes: usize, out_d_ptr: *mut *mut c_void) -> EtcStatus;
    pub fn etc_free(rt: *mut EtcRuntime, d_ptr: *mut c_void) -> EtcStatus;
    pub fn etc_upload(rt: *mut EtcRuntime, d_dst: *mut c_void, h_src: *const c_void, bytes: usize) -> EtcStatus;
    pub fn etc_download(rt: *mut EtcRuntime, h_dst: *mut c_void, d_src: *const c_void, bytes: usize) -> EtcStatus;
    pub fn etc_encoded_row_bytes(codec: c_int, columns: i64, out_bytes: *mut i64) -> EtcStatus;
    pub fn etc_dequantize_into(
        rt: *mut EtcRuntime,
        codec: c_int,
        d_packed: *const c_void,
        rows: i64,
        columns: i64,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_quantize_into(
        rt: *mut EtcRuntime,
        codec: c_int,
        d_x: *const f32,
        rows: i64,
        columns: i64,
        d_packed: *mut c_void,
    ) -> EtcStatus;
    pub fn etc_qlinear_requirements(
        codec: c_int,
        vectors: i64,
        rows: i64,
        columns: i64,
        out_bytes: *mut usize,
        scratch_bytes: *mut usize,
    ) -> EtcStatus;
    pub fn etc_qlinear_into(
        rt: *mut EtcRuntime,
        codec: c_int,
        d_x: *const f32,
        vectors: i64,
        columns: i64,
        d_weight: *const c_void,
        rows: i64,
        d_bias: *const f32,
        d_out: *mut f32,
        cancelled: *const c_int,
    ) -> EtcStatus;
    pub fn etc_qweight_create(
        rt: *mut EtcRuntime,
        codec: c_int,
        parts: *const *const c_void,
        part_rows: *const i64,
        n_parts: c_int,
        columns: i64,
        interleave8: c_int,
        on_device: c_int,
        out: *mut *mut EtcQweight,
    ) -> EtcStatus;
    pub fn etc_qweight_destroy(w: *mut EtcQweight) -> EtcStatus;
    pub fn etc_qweight_shape(
        w: *const EtcQweight,
        rows: *mut i64,
        columns: *mut i64,
        codec: *mut c_int,
        device_bytes: *mut u64,
    ) -> EtcStatus;
    pub fn etc_qlinear_tiled_scratch_bytes(
        w: *const EtcQweight,
        vectors: i64,
        scratch_bytes: *mut usize,
    ) -> EtcStatus;
    pub fn etc_qlinear_tiled_into(
        rt: *mut EtcRuntime,
        w: *const EtcQweight,
        d_x: *const f32,
        vectors: i64,
        d_bias: *const f32,
        d_residual: *const f32,
        epilogue: c_int,
        d_out: *mut f32,
        d_scratch: *mut c_void,
        scratch_bytes: usize,
    ) -> EtcStatus;
    pub fn etc_qlinear_tiled_static_max_bytes(max_bytes: *mut usize) -> EtcStatus;
    pub fn etc_qlinear_tiled_static_into(
        rt: *mut EtcRuntime,
        w: *const EtcQweight,
        d_x: *const f32,
        vectors: i64,
        d_bias: *const f32,
        d_residual: *const f32,
        epilogue: c_int,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_qembedding_into(
        rt: *mut EtcRuntime,
        codec: c_int,
        d_indexes: *const c_void,
        index_dtype: c_int,
        count: i64,
        d_weight: *const c_void,
        rows: i64,
        columns: i64,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_linear_f32_into(
        rt: *mut EtcRuntime,
        d_x: *const f32,
        m: i64,
        k: i64,
        d_w: *const f32,
        n: i64,
        d_bias: *const f32,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_rmsnorm_into(
        rt: *mut EtcRuntime,
        d_x: *const f32,
        d_weight: *const f32,
        eps: f64,
        rows: i64,
        n: i64,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_rope_into(
        rt: *mut EtcRuntime,
        d_x: *const f32,
        d_offsets: *const i64,
        n_offsets: i64,
        theta: f64,
        layout: c_int,
        batch: i64,
        heads: i64,
        steps: i64,
        head_dim: i64,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_swiglu_into(
        rt: *mut EtcRuntime,
        d_gate: *const f32,
        d_up: *const f32,
        n: i64,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_add_into(rt: *mut EtcRuntime, d_a: *const f32, d_b: *const f32, n: i64, d_out: *mut f32) -> EtcStatus;
    pub fn etc_argmax_into(
        rt: *mut EtcRuntime,
        d_logits: *const f32,
        rows: i64,
        vocab: i64,
        d_tokens: *mut u32,
    ) -> EtcStatus;
    pub fn etc_sample_rows_into(
        rt: *mut EtcRuntime,
        d_logits: *const f32,
        rows: i64,
        vocab: i64,
        temperature: f64,
        top_k: i64,
        top_p: f64,
        seed: u64,
        counter: u64,
        d_seeds: *const u64,
        d_counters: *const u64,
        d_tokens: *mut u32,
    ) -> EtcStatus;
    pub fn etc_sample_row(
        rt: *mut EtcRuntime,
        d_logits: *const f32,
        vocab: i64,
        temperature: f64,
        top_k: i64,
        top_p: f64,
        seed: u64,
        counter: u64,
        out_token: *mut u32,
    ) -> EtcStatus;
    pub fn etc_pool_create(
        rt: *mut EtcRuntime,
        layers: c_int,
        kv_heads: c_int,
        head_dim: c_int,
        max_tokens: c_int,
        block_size: c_int,
        dtype: c_int,
        out: *mut *mut EtcPool,
    ) -> EtcStatus;
    pub fn etc_pool_destroy(pool: *mut EtcPool) -> EtcStatus;
    pub fn etc_pool_stats(
        pool: *mut EtcPool,
        capacity: *mut u32,
        free_blocks: *mut u32,
        cached_blocks: *mut u32,
    ) -> EtcStatus;
    pub fn etc_pool_state_bytes(
        layers: i64,
        max_tokens: i64,
        kv_heads: i64,
        head_dim: i64,
        dtype: c_int,
        out_bytes: *mut i64,
    ) -> EtcStatus;
    pub fn etc_pool_read_rows(
        pool: *mut EtcPool,
        layer: c_int,
        which: c_int,
        h_rows: *const u32,
        n: i64,
        h_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_seq_create(pool: *mut EtcPool, out: *mut *mut EtcSeq) -> EtcStatus;
    pub fn etc_seq_release(seq: *mut EtcSeq) -> EtcStatus;
    pub fn etc_seq_destroy(seq: *mut EtcSeq) -> EtcStatus;
    pub fn etc_seq_cursor(seq: *mut EtcSeq, out_cursor: *mut u32) -> EtcStatus;
    pub fn etc_seq_prefill_match(
        seq: *mut EtcSeq,
        h_tokens: *const u32,
        count: i64,
        out_matched: *mut u32,
    ) -> EtcStatus;
    pub fn etc_seq_blocks(
        seq: *mut EtcSeq,
        h_out: *mut u32,
        capacity: i64,
        out_count: *mut i64,
        out_head: *mut i64,
    ) -> EtcStatus;
    pub fn etc_kv_attention_into(
        rt: *mut EtcRuntime,
        pool: *mut EtcPool,
        layer: c_int,
        seqs: *const *mut EtcSeq,
        batch: c_int,
        active: c_int,
        advance: c_int,
        d_q: *const f32,
        d_k: *const f32,
        d_v: *const f32,
        q_heads: c_int,
        tokens: c_int,
        scale: f64,
        op_window: i64,
        pool_window: i64,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_kv_append_into(
        rt: *mut EtcRuntime,
        pool: *mut EtcPool,
        layer: c_int,
        seqs: *const *mut EtcSeq,
        batch: c_int,
        active: c_int,
        advance: c_int,
        d_k: *const f32,
        d_v: *const f32,
        tokens: c_int,
        pool_window: i64,
    ) -> EtcStatus;
    pub fn etc_kv_attention_decode_into(
        rt: *mut EtcRuntime,
        pool: *mut EtcPool,
        layer: c_int,
        seqs: *const *mut EtcSeq,
        batch: c_int,
        active: c_int,
        d_q: *const f32,
        d_k: *const f32,
        d_v: *const f32,
        q_heads: c_int,
        scale: f64,
        op_window: i64,
        pool_window: i64,
        d_out: *mut f32,
    ) -> EtcStatus;
    pub fn etc_seq_commit(seq: *mut EtcSeq, h_tokens: *const u32, advance: c_int, eviction_start: i64) -> EtcStatus;
    pub fn etc_seq_rollback(seq: *mut EtcSeq, frontier: i64) -> EtcStatus;
    pub fn etc_seq_frontier(seq: *mut EtcSeq, out_frontier: *mut i64) -> EtcStatus;
    pub fn etc_gguf_open(path: *const c_char, cancelled: *const c_int, out: *mut *mut EtcGguf) -> EtcStatus;
    pub fn etc_gguf_close(file: *mut EtcGguf) -> EtcStatus;
    pub fn etc_gguf_summary(
        file: *const EtcGguf,
        architecture: *mut *const c_char,
        metadata_count: *mut i64,
        tensor_count: *mut i64,
    ) -> EtcStatus;
    pub fn etc_gguf_metadata(
        file: *const EtcGguf,
        index: i64,
        key: *mut *const c_char,
        value_type: *mut c_int,
        element_type: *mut c_int,
        count: *mut i64,
        integer_bits: *mut u64,
        real: *mut f64,
        string: *mut *const c_char,
    ) -> EtcStatus;
    pub fn etc_gguf_tensor(
        file: *const EtcGguf,
        index: i64,
        name: *mut *const c_char,
        codec: *mut c_int,
        rank: *mut c_int,
        logical_shape4: *mut i64,
        physical_shape4: *mut i64,
        data_offset: *mut u64,
        byte_len: *mut u64,
    ) -> EtcStatus;
    pub fn etc_gguf_find_tensor(file: *const EtcGguf, name: *const c_char, index: *mut i64) -> EtcStatus;
    pub fn etc_gguf_read_tensor_into(
        file: *const EtcGguf,
        index: i64,
        h_dst: *mut c_void,
        dst_bytes: u64,
        cancelled: *const c_int,
    ) -> EtcStatus;
    pub fn etc_gguf_load_tensor_device(
        rt: *mut EtcRuntime,
        file: *const EtcGguf,
        index: i64,
        d_dst: *mut c_void,
        dst_bytes: u64,
        cancelled: *const c_int,
    ) -> EtcStatus;
    pub fn etc_tp_unique_id(out_id_128_bytes: *mut u8) -> EtcStatus;
    pub fn etc_decoder_set_tensor_parallel(
        dec: *mut EtcDecoder,
        rank: c_int,
        world: c_int,
        id_128_bytes: *const u8,
    ) -> EtcStatus;
    pub fn etc_decoder_tp_peer_export(dec: *mut EtcDecoder, out_handle_64_bytes: *mut u8) -> EtcStatus;
    pub fn etc_decoder_tp_peer_import(dec: *mut EtcDecoder, handles_world_x_64_bytes: *const u8) -> EtcStatus;
    pub fn etc_decoder_tp_region(
        dec: *mut EtcDecoder,
        out_region: *mut *mut c_void,
        out_bytes: *mut usize,
    ) -> EtcStatus;
    pub fn etc_decoder_tp_peer_attach(dec: *mut EtcDecoder, regions_world: *const *mut c_void) -> EtcStatus;
    pub fn etc_decoder_set_wait_limit(dec: *mut EtcDecoder, cycles: i64) -> EtcStatus;
    pub fn etc_decoder_set_head_shard(dec: *mut EtcDecoder, vocab_global: i64, first_row: i64) -> EtcStatus;
    pub fn etc_peer_region_bytes(capacity: i64, world: c_int) -> usize;
    pub fn etc_peer_allreduce_into(
        rt: *mut EtcRuntime,
        rank: c_int,
        world: c_int,
        regions: *const *mut c_void,
        capacity: i64,
        buffer: c_int,
        d_partial: *const f32,
        d_hidden: *mut f32,
        count: i64,
        two_shot: c_int,
        wait_cycles: i64,
    ) -> EtcStatus;
    pub fn etc_paged_attention_into(
        rt: *mut EtcRuntime,
        pool: *mut EtcPool,
        layer: c_int,
        d_lanes: *const EtcLane,
        d_tables: *const c_int,
        batch: c_int,
        max_pages: c_int,
        d_q: *const f32,
        q_heads: c_int,
        scale: f64,
        op_window: i64,
        d_out: *mut f32,
        d_scratch: *mut c_void,
        scratch_bytes: usize,
    ) -> EtcStatus;
    pub fn etc_kv_attention_plan(
        batch: c_int,
        q_heads: c_int,
        kv_heads: c_int,
        head_dim: c_int,
        attended_pages: c_int,
        sm_count: c_int,
        splits: *mut c_int,
        pages_per_split: *mut c_int,
        partial_bytes: *mut usize,
    ) -> EtcStatus;
    pub fn etc_decoder_attention_reserve(
        config: *const EtcDecoderConfig,
        max_advance: c_int,
        sm_count: c_int,
        max_blocks: *mut c_int,
        partial_bytes: *mut usize,
    ) -> EtcStatus;
    pub fn etc_decoder_create(
        rt: *mut EtcRuntime,
        config: *const EtcDecoderConfig,
        out: *mut *mut EtcDecoder,
    ) -> EtcStatus;
    pub fn etc_decoder_destroy(dec: *mut EtcDecoder) -> EtcStatus;
    pub fn etc_decoder_set_weight(
        dec: *mut EtcDecoder,
        slot: c_int,
        layer: c_int,
        codec: c_int,
        h_data: *const c_void,
        rows: i64,
        columns: i64,
    ) -> EtcStatus;
    pub fn etc_decoder_set_weight_device(
        dec: *mut EtcDecoder,
        slot: c_int,
        layer: c_int,
        codec: c_int,
        d_data: *const c_void,
        rows: i64,
        columns: i64,
    ) -> EtcStatus;
    pub fn etc_decoder_set_max_advance(dec: *mut EtcDecoder, max_advance: c_int) -> EtcStatus;
    pub fn etc_decoder_finalize(dec: *mut EtcDecoder) -> EtcStatus;
    pub fn etc_decoder_execute(
        dec: *mut EtcDecoder,
        pool: *mut EtcPool,
        seqs: *const *mut EtcSeq,
        active: c_int,
        h_tokens: *const u32,
        advance: c_int,
        h_logits: *mut f32,
        cancelled: *const c_int,
    ) -> EtcStatus;
    pub fn etc_decoder_execute_sampled(
        dec: *mut EtcDecoder,
        pool: *mut EtcPool,
        seqs: *const *mut EtcSeq,
        active: c_int,
        h_tokens: *const u32,
        advance: c_int,
        h_out_tokens: *mut u32,
        cancelled: *const c_int,
    ) -> EtcStatus;
    pub fn etc_decoder_generate_greedy(
        dec: *mut EtcDecoder,
        pool: *mut EtcPool,
        seqs: *const *mut EtcSeq,
        active: c_int,
        h_first_tokens: *const u32,
        steps: c_int,
        h_out_tokens: *mut u32,
        out_device_ms: *mut f32,
    ) -> EtcStatus;
    pub fn etc_decoder_diagnostics(
        dec: *mut EtcDecoder,
        launches_per_step: *mut c_int,
        weight_bytes: *mut u64,
        workspace_bytes: *mut u64,
    ) -> EtcStatus;
}
