/*
 * et_cuda.h — C ABI of the B200 (sm_100a) CUDA backend for effect-torch's compiled-inference
 * hot path: paged-KV-cache batched decode over GGUF block-quantized weights.
 *
 * This is the surface a `crates/runtime-cuda` crate (and through it a napi addon and the
 * `@effect-torch/backend-cuda` Runtime Layer) binds. It sits below graph lowering, where the
 * reference's CPU backend keeps its `*_requirements` planners and allocation-free `*_into`
 * kernels (crates/runtime-cpu/src/lib.rs:5-11). File:line citations name the reference
 * interface each entry point replaces; paths are relative to the reference project root.
 *
 * Conventions
 *   - Every function returns an etc_status. On failure etc_last_error_message() (thread-local)
 *     holds the text; the texts the reference's callers and tests match on are kept verbatim
 *     ("operation aborted", "pool exhausted", "exceeds pool capacity", "is outside 0..", ...).
 *   - The status classes mirror BackendError (crates/runtime/src/error.rs:25-68).
 *   - Handles are opaque. Inputs are borrowed for the duration of the call, outputs are written
 *     into caller-provided buffers, release is idempotent (packages/core/src/Runtime.ts:14-24).
 *   - Pointers named d_* are device pointers of the runtime's device; h_* are host pointers.
 *     All tensors are dense row-major. No torch or C++ types cross this boundary.
 *   - Launches go to the runtime's stream (etc_runtime_stream); `*_into` calls are
 *     asynchronous unless stated; device-detected problems (index out of range, non-finite
 *     logit) are reported through a status word read at the next synchronising call.
 *   - There is no CPU fallback: a call that cannot run on the device fails.
 *   - Threads: different runtimes may be driven from different threads freely. Calls on ONE runtime (and on the pools,
 *     weights and decoders made from it) share its stream, status word and staging buffers: the host serialises them,
 *     as the reference's addon does with one worker per executable invocation. Sequences carry their own run lock, so
 *     two steps over disjoint sequences are ordered by the caller only through the runtime they share.
 */
#ifndef ET_CUDA_H
#define ET_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ETC_API __attribute__((visibility("default")))
#else
#define ETC_API
#endif

/* ---- status (crates/runtime/src/error.rs:25-68, packages/core/src/Runtime.ts:129-143) ---- */
typedef enum etc_status {
  ETC_OK = 0,
  ETC_UNAVAILABLE = 1,    /* backend-unavailable / device-unavailable */
  ETC_UNSUPPORTED = 2,    /* unsupported-operation / dtype / layout / placement */
  ETC_INVALID_HANDLE = 3, /* invalid-handle / foreign-handle */
  ETC_COMPILATION = 4,    /* compilation-failed (plan construction, geometry validation) */
  ETC_EXECUTION = 5,      /* execution-failed */
  ETC_TRANSFER = 6,       /* transfer-failed */
  ETC_CANCELLED = 7,      /* cancelled: message is exactly "operation aborted" */
  ETC_CLOSED = 8,         /* closed-runtime */
  ETC_INVALID_ARGUMENT = 9 /* napi Status::InvalidArg class (argument validation before any work) */
} etc_status;

/* Block codecs: values are the GGML tensor type codes stored in a GGUF tensor catalog
 * (crates/runtime/src/gguf.rs:279-291 accepts 0 and 10..14; 2 and 8 are added by this backend). */
typedef enum etc_codec {
  ETC_CODEC_F32 = 0,
  ETC_CODEC_Q4_0 = 2,
  ETC_CODEC_Q8_0 = 8,
  ETC_CODEC_Q2_K = 10,
  ETC_CODEC_Q3_K = 11,
  ETC_CODEC_Q4_K = 12,
  ETC_CODEC_Q5_K = 13,
  ETC_CODEC_Q6_K = 14
} etc_codec;

/* KV tiers (crates/runtime-cpu/src/pool.rs:20-25). */
typedef enum etc_kv_dtype { ETC_KV_F32 = 0, ETC_KV_F16 = 1, ETC_KV_BF16 = 2, ETC_KV_U8 = 3 } etc_kv_dtype;

/* RotaryLayout (crates/runtime-cpu/src/composed.rs:2714-2717). */
typedef enum etc_rope_layout { ETC_ROPE_HALF_SPLIT = 0, ETC_ROPE_INTERLEAVED_PAIRS = 1 } etc_rope_layout;

typedef enum etc_index_dtype { ETC_INDEX_U32 = 0, ETC_INDEX_I64 = 1 } etc_index_dtype;

typedef struct etc_runtime etc_runtime;
typedef struct etc_pool etc_pool;
typedef struct etc_seq etc_seq;
typedef struct etc_qweight etc_qweight;
typedef struct etc_decoder etc_decoder;

#define ETC_NO_WINDOW (-1)

/* ------------------------------------------------------------------------------------------
 * Runtime. Replaces the per-backend `makeRuntime()` / `isAvailable()` of the napi addon
 * (packages/backend-cpu/src/index.ts:27, packages/backend-cpu/src/internal/native-addon.ts:430-445).
 * ------------------------------------------------------------------------------------------ */
ETC_API const char* etc_last_error_message(void);
ETC_API const char* etc_version(void);
/* Number of usable CUDA devices; 0 (with ETC_OK) when there is none. */
ETC_API etc_status etc_device_count(int* out_count);
ETC_API etc_status etc_runtime_create(int device_ordinal, etc_runtime** out);
ETC_API etc_status etc_runtime_destroy(etc_runtime* rt);
/* The runtime's CUDA stream as a cudaStream_t value. */
ETC_API etc_status etc_runtime_stream(etc_runtime* rt, void** out_stream);
/* Waits for the stream and reports any device-side status word raised since the last call. */
ETC_API etc_status etc_runtime_synchronize(etc_runtime* rt);
/* Count of kernels launched by this library on this runtime since creation. */
ETC_API etc_status etc_runtime_launch_count(etc_runtime* rt, uint64_t* out);
/* Bytes of device memory currently held by this runtime's handles (the analogue of
 * external_memory_bytes, crates/runtime-cpu/src/napi/mod.rs:2373-2376). */
ETC_API etc_status etc_runtime_memory_bytes(etc_runtime* rt, uint64_t* out);

/* Capabilities (crates/runtime/src/backend.rs:168-206: the dtypes and optional features a backend reports).
 * dtype_mask has bit i set for etc_dtype_bit i; feature_mask bit 0 = compilation, bit 1 = asynchronous execution,
 * bit 2 = unified memory (never set: device memory is separate). device_name receives a NUL-terminated copy. */
typedef enum etc_dtype_bit {
  ETC_DTYPE_F32 = 0, ETC_DTYPE_F64 = 1, ETC_DTYPE_F16 = 2, ETC_DTYPE_BF16 = 3, ETC_DTYPE_U8 = 4, ETC_DTYPE_U32 = 5, ETC_DTYPE_I64 = 6
} etc_dtype_bit;
typedef struct etc_capabilities {
  uint32_t dtype_mask;
  uint32_t feature_mask;
  int device_ordinal;
  int sm_count;
  int compute_major, compute_minor;
  uint64_t device_memory_bytes;
  char device_name[128];
} etc_capabilities;
ETC_API etc_status etc_runtime_capabilities(etc_runtime* rt, etc_capabilities* out);

/* Device buffers (NativeTensor storage; crates/runtime/src/backend.rs:215-221). */
ETC_API etc_status etc_alloc(etc_runtime* rt, size_t bytes, void** out_d_ptr);
ETC_API etc_status etc_free(etc_runtime* rt, void* d_ptr);
ETC_API etc_status etc_upload(etc_runtime* rt, void* d_dst, const void* h_src, size_t bytes);     /* synchronous */
ETC_API etc_status etc_download(etc_runtime* rt, void* h_dst, const void* d_src, size_t bytes);   /* synchronous; readback */

/* ------------------------------------------------------------------------------------------
 * Block-quantized weights.
 * ------------------------------------------------------------------------------------------ */
/* GgmlKQuant::encoded_row_bytes (crates/runtime/src/gguf.rs:245-250) extended to 32-value codecs.
 * ETC_COMPILATION "logical row width {columns} is invalid for {codec}" when columns is not a
 * whole number of blocks. */
ETC_API etc_status etc_encoded_row_bytes(etc_codec codec, int64_t columns, int64_t* out_bytes);

/* Decode packed rows to f32, bit-exact with decode_block (crates/runtime-cpu/src/quantized.rs:90-261).
 * d_packed is an exact contiguous [rows, encoded_row_bytes] u8 tensor. */
ETC_API etc_status etc_dequantize_into(etc_runtime* rt, etc_codec codec, const void* d_packed, int64_t rows,
                                       int64_t columns, float* d_out);

/* Quantize f32 [rows, columns] to Q4_0 or Q8_0 packed rows (the reference has no weight quantizer;
 * semantics are documented with the kernel). */
ETC_API etc_status etc_quantize_into(etc_runtime* rt, etc_codec codec, const float* d_x, int64_t rows, int64_t columns,
                                     void* d_packed);

/* linear_requirements (quantized.rs:297-336): validates geometry, returns output bytes and the
 * scratch bytes etc_qlinear_into needs for these sizes. */
ETC_API etc_status etc_qlinear_requirements(etc_codec codec, int64_t vectors, int64_t rows, int64_t columns,
                                            size_t* out_bytes, size_t* scratch_bytes);

/* linear_into (quantized.rs:419-499): out[v,row] = sum_k x[v,k] * deq(W[row,k]) (+ bias[row]).
 * d_x f32 [vectors, columns]; d_weight raw GGUF packed [rows, encoded_row_bytes]; d_out f32
 * [vectors, rows]. Works for every codec on the raw layout. `cancelled` (host flag, may be NULL)
 * is polled before the launch: ETC_CANCELLED "operation aborted". */
ETC_API etc_status etc_qlinear_into(etc_runtime* rt, etc_codec codec, const float* d_x, int64_t vectors,
                                    int64_t columns, const void* d_weight, int64_t rows, const float* d_bias,
                                    float* d_out, const volatile int* cancelled);

/* Constant weights (ExecutableCompileOptions.constantWeights, packages/core/src/Runtime.ts:249-256):
 * a packed matrix retained by the backend in a device-friendly tiling. `parts` are raw packed row
 * ranges concatenated along rows (e.g. q,k,v); interleave8 != 0 interleaves two equal parts in groups
 * of 8 rows (gate/up), which lets the linear's epilogue compute silu(gate)*up.
 * Q4_0 / Q8_0 (columns a multiple of 64): same bytes, same dequantised values, reordered.
 * Q3_K / Q4_K / Q5_K / Q6_K (columns a multiple of 256): every 256-value block is re-cut into eight
 * 32-value blocks whose effective scales (d*sc) and minima (dmin*m) are rounded to f16 once, at load
 * (20 B per 32 values for Q4_K, 36 B for the others). Q2_K and F32 are refused (ETC_UNSUPPORTED): they
 * run through etc_qlinear_into on the raw layout.
 * Pointers are device pointers when on_device != 0, host pointers otherwise. */
ETC_API etc_status etc_qweight_create(etc_runtime* rt, etc_codec codec, const void* const* parts,
                                      const int64_t* part_rows, int n_parts, int64_t columns, int interleave8,
                                      int on_device, etc_qweight** out);
ETC_API etc_status etc_qweight_destroy(etc_qweight* w);
ETC_API etc_status etc_qweight_shape(const etc_qweight* w, int64_t* rows, int64_t* columns, etc_codec* codec,
                                     uint64_t* device_bytes);

typedef enum etc_epilogue {
  ETC_EPILOGUE_NONE = 0,     /* out = x W^T (+bias) */
  ETC_EPILOGUE_RESIDUAL = 1, /* out = residual + x W^T (+bias): the residual add that follows o/down projections */
  ETC_EPILOGUE_SWIGLU = 2    /* weight built with interleave8: out[v,i] = silu(gate_i) * up_i, out is [vectors, rows/2] */
} etc_epilogue;

/* Scratch bytes the tiled linear needs for `vectors` input rows (split-K partial sums). */
ETC_API etc_status etc_qlinear_tiled_scratch_bytes(const etc_qweight* w, int64_t vectors, size_t* scratch_bytes);

/* Tensor-core linear over a retained weight. d_x f32 [vectors, columns]; d_out f32;
 * d_scratch must hold etc_qlinear_tiled_scratch_bytes (NULL lets the runtime use its own workspace). */
ETC_API etc_status etc_qlinear_tiled_into(etc_runtime* rt, const etc_qweight* w, const float* d_x, int64_t vectors,
                                          const float* d_bias, const float* d_residual, etc_epilogue epilogue,
                                          float* d_out, void* d_scratch, size_t scratch_bytes);

/* The same linear with its scratch in a fixed 16 MiB device array inside the library: the call allocates nothing,
 * neither device nor pinned memory, for callers that must not allocate while they run. No counterpart in the
 * reference, whose backends allocate per operation. Results equal etc_qlinear_tiled_into's bit for bit when the call's
 * scratch (etc_qlinear_tiled_scratch_bytes) fits etc_qlinear_tiled_static_max_bytes; a longer call runs 256 vectors at
 * a time, whose split plans can differ from the one-pass plan (same values to the linear's tolerance), and is rejected
 * with ETC_INVALID_ARGUMENT only when a 256-vector slice does not fit either (the message gives both sizes). The array's 16 MiB are reserved on a device when etc_runtime_create runs for it (that is when its device
 * address is looked up, which loads the module holding it), so create the runtime before dividing the remaining
 * device memory among your own pools; the entry point looks the address up again only if that step was skipped, and
 * that look-up should not happen during a stream capture. All calls on a device share the array: calls that overlap in
 * time race, serialise them. Nothing in the array needs to be zero. */
ETC_API etc_status etc_qlinear_tiled_static_max_bytes(size_t* max_bytes);
ETC_API etc_status etc_qlinear_tiled_static_into(etc_runtime* rt, const etc_qweight* w, const float* d_x, int64_t vectors,
                                                 const float* d_bias, const float* d_residual, etc_epilogue epilogue,
                                                 float* d_out);

/* embedding_into (quantized.rs:546-616): decode rows selected by u32/i64 indexes. An index that is
 * negative or >= rows is reported at the next synchronising call as ETC_EXECUTION
 * "quantized_embedding: index {i} is outside 0..{rows}". codec F32 gathers dense rows. */
ETC_API etc_status etc_qembedding_into(etc_runtime* rt, etc_codec codec, const void* d_indexes,
                                       etc_index_dtype index_dtype, int64_t count, const void* d_weight, int64_t rows,
                                       int64_t columns, float* d_out);

/* ------------------------------------------------------------------------------------------
 * Dense / elementwise ops of the decode graph.
 * ------------------------------------------------------------------------------------------ */
/* Dense linearRows (packages/core/src/Tensor.ts:5242-5245 -> crates/runtime-cpu/src/matmul.rs:192-231):
 * out[m,n] = fma chain over k of x[m,k] * W[n,k], sequential in k (bit-exact with the reference). */
ETC_API etc_status etc_linear_f32_into(etc_runtime* rt, const float* d_x, int64_t m, int64_t k, const float* d_w,
                                       int64_t n, const float* d_bias, float* d_out);
/* rms_norm_forward_into (crates/runtime-cpu/src/composed.rs:1457-1533). d_weight may be NULL. */
ETC_API etc_status etc_rmsnorm_into(etc_runtime* rt, const float* d_x, const float* d_weight, double eps, int64_t rows,
                                    int64_t n, float* d_out);
/* rotary_forward_into with per-lane cursors (composed.rs:2683-2775; crates/runtime-cpu/src/napi/mod.rs:2830-2838).
 * d_x/d_out f32 [batch, heads, steps, head_dim]; d_offsets i64 [n_offsets], n_offsets is 1 or batch. */
ETC_API etc_status etc_rope_into(etc_runtime* rt, const float* d_x, const int64_t* d_offsets, int64_t n_offsets,
                                 double theta, etc_rope_layout layout, int64_t batch, int64_t heads, int64_t steps,
                                 int64_t head_dim, float* d_out);
/* silu(gate) * up with sigmoid(x) = tanh(x/2)/2 + 1/2 (packages/core/src/Tensor.ts:1240-1245, 1537-1540). */
ETC_API etc_status etc_swiglu_into(etc_runtime* rt, const float* d_gate, const float* d_up, int64_t n, float* d_out);
ETC_API etc_status etc_add_into(etc_runtime* rt, const float* d_a, const float* d_b, int64_t n, float* d_out);
/* Greedy branch of sample_logits (crates/runtime/src/sampling.rs:88-105): first index of the maximum per
 * row. A non-finite logit is reported at the next synchronising call as ETC_EXECUTION
 * "sample: logit {i} is not finite". d_tokens u32 [rows]. */
ETC_API etc_status etc_argmax_into(etc_runtime* rt, const float* d_logits, int64_t rows, int64_t vocab,
                                   uint32_t* d_tokens);
/* sample_logits (crates/runtime/src/sampling.rs:80-206) on the device, one CTA per logits row: temperature 0 = greedy;
 * otherwise candidates in (value descending, token ascending) order, the first top_k of them (0 = all), weights
 * exp((value - max) / temperature), the smallest prefix holding top_p of the weight, and the candidate at which the
 * splitmix64 unit of (seed, counter) x total is used up; without top-k and top-p the walk is in token order. Row r draws
 * with (d_seeds[r], d_counters[r]) when those device arrays are given, else with the scalars. Asynchronous; argument
 * errors carry the reference's messages, a non-finite logit surfaces at the next synchronising call. The sums are f64 as
 * in the reference but associated differently, so a token can differ only when the draw (or the top-p threshold) lies
 * within about vocab x 2^-52 (relative) of a candidate's boundary. */
ETC_API etc_status etc_sample_rows_into(etc_runtime* rt, const float* d_logits, int64_t rows, int64_t vocab, double temperature,
                                        int64_t top_k, double top_p, uint64_t seed, uint64_t counter, const uint64_t* d_seeds,
                                        const uint64_t* d_counters, uint32_t* d_tokens);
/* One row, synchronous, token returned to the host. */
ETC_API etc_status etc_sample_row(etc_runtime* rt, const float* d_logits, int64_t vocab, double temperature,
                                  int64_t top_k, double top_p, uint64_t seed, uint64_t counter, uint32_t* out_token);

/* ------------------------------------------------------------------------------------------
 * Paged KV pool and sequences (NativeKvPool / NativeKvSequence,
 * crates/runtime-cpu/src/napi/mod.rs:3632-3947; native-addon.ts:193-220).
 * ------------------------------------------------------------------------------------------ */
ETC_API etc_status etc_pool_create(etc_runtime* rt, int layers, int kv_heads, int head_dim, int max_tokens,
                                   int block_size, etc_kv_dtype dtype, etc_pool** out);
ETC_API etc_status etc_pool_destroy(etc_pool* pool);
/* capacity / freeBlocks / cachedBlocks getters (napi/mod.rs:3753-3766). */
ETC_API etc_status etc_pool_stats(etc_pool* pool, uint32_t* capacity, uint32_t* free_blocks, uint32_t* cached_blocks);
/* KvStateSchema::referenced_state_bytes for the KV part (napi/mod.rs:1921-1980). */
ETC_API etc_status etc_pool_state_bytes(int64_t layers, int64_t max_tokens, int64_t kv_heads, int64_t head_dim,
                                        etc_kv_dtype dtype, int64_t* out_bytes);
/* Debug/test access: read logical token rows of one layer slab back as f32 [n, kv_heads*head_dim]
 * in the reference's row order (row = token slot index = block*block_size + offset). which: 0 K, 1 V.
 * The u8 tier returns dequantised values ((code-128)*scale, napi/mod.rs:3474-3476). Synchronous. */
ETC_API etc_status etc_pool_read_rows(etc_pool* pool, int layer, int which, const uint32_t* h_rows, int64_t n,
                                      float* h_out);

ETC_API etc_status etc_seq_create(etc_pool* pool, etc_seq** out);      /* makeSequence() */
ETC_API etc_status etc_seq_release(etc_seq* seq);                      /* release(): idempotent, returns blocks */
ETC_API etc_status etc_seq_destroy(etc_seq* seq);                      /* finalize/drop: releases, then frees the handle */
ETC_API etc_status etc_seq_cursor(etc_seq* seq, uint32_t* out_cursor); /* cursor getter */
/* prefillMatch(tokens) (napi/mod.rs:3874-3946): reuse cached whole blocks by chained FNV-1a hash. */
ETC_API etc_status etc_seq_prefill_match(etc_seq* seq, const uint32_t* h_tokens, int64_t count, uint32_t* out_matched);
/* The sequence's block list (page table) from its first live block; for tests of page-table parity. */
ETC_API etc_status etc_seq_blocks(etc_seq* seq, uint32_t* h_out, int64_t capacity, int64_t* out_count, int64_t* out_head);

/* kv_attention_into (napi/mod.rs:3320-3565) for one KvAttention node outside a compiled decoder:
 * page allocation (kv_prepare), scatter of the `advance` new K/V rows of each active lane, then
 * attention over the block table. d_q f32 [batch, q_heads, tokens, head_dim], d_k/d_v f32
 * [batch, kv_heads, tokens, head_dim], d_out like d_q (zero for lanes >= active). `advance` is the
 * number of live rows per lane (1..tokens). op_window / pool_window: ETC_NO_WINDOW or a window.
 * Synchronous with respect to host state: block lists are updated before return; the cursor is NOT
 * advanced (call etc_seq_commit / etc_seq_rollback, the transaction of executable.rs:4593-4665). */
ETC_API etc_status etc_kv_attention_into(etc_runtime* rt, etc_pool* pool, int layer, etc_seq* const* seqs, int batch,
                                         int active, int advance, const float* d_q, const float* d_k, const float* d_v,
                                         int q_heads, int tokens, double scale, int64_t op_window, int64_t pool_window,
                                         float* d_out);
/* The scatter half of kv_attention_into alone (napi/mod.rs:3397-3459): page allocation plus the write of
 * the `advance` new K/V rows of each active lane. d_k/d_v f32 [batch, kv_heads, tokens, head_dim]. */
ETC_API etc_status etc_kv_append_into(etc_runtime* rt, etc_pool* pool, int layer, etc_seq* const* seqs, int batch,
                                      int active, int advance, const float* d_k, const float* d_v, int tokens,
                                      int64_t pool_window);
/* kv_attention_into for one-token decode steps on the tensor-core flash-decoding kernel (f16/bf16 pools,
 * 16-token pages, head dim 64/128): d_q f32 [batch, q_heads, head_dim], d_k/d_v f32 [batch, kv_heads,
 * head_dim] (may both be NULL when the step's rows were already appended), d_out like d_q. Same page
 * allocation, masking and window rules as etc_kv_attention_into; results within the f16 tolerance. */
ETC_API etc_status etc_kv_attention_decode_into(etc_runtime* rt, etc_pool* pool, int layer, etc_seq* const* seqs,
                                                int batch, int active, const float* d_q, const float* d_k,
                                                const float* d_v, int q_heads, double scale, int64_t op_window,
                                                int64_t pool_window, float* d_out);
/* Commit: note tokens (block hashes), evict window-dead blocks below `eviction_start` (pass 0 for none),
 * cursor += advance (napi/mod.rs:2844-2877, 4511-4518). */
ETC_API etc_status etc_seq_commit(etc_seq* seq, const uint32_t* h_tokens, int advance, int64_t eviction_start);
/* Rollback: unreference blocks pushed since `frontier` blocks, cursor untouched (napi/mod.rs:2879-2895). */
ETC_API etc_status etc_seq_rollback(etc_seq* seq, int64_t frontier);
ETC_API etc_status etc_seq_frontier(etc_seq* seq, int64_t* out_frontier);

/* ------------------------------------------------------------------------------------------
 * Compiled decoder: the stateful Executable of a Llama-shaped model (compile + Executable.execute /
 * executeSampled, native-addon.ts:43-56, 252-257; crates/runtime-cpu/src/napi/mod.rs:4150-4522).
 * ------------------------------------------------------------------------------------------ */
typedef struct etc_decoder_config {
  int layers, d_model, q_heads, kv_heads, head_dim, ffn, vocab;
  double rms_eps, rope_theta;
  int rope_layout;      /* etc_rope_layout */
  int64_t window;       /* ETC_NO_WINDOW, or a sliding window applied by every attention layer */
  int batch;            /* compiled batch (KvStateSchema.batch) */
  int max_tokens;       /* KvStateSchema.max_tokens; must match the pool */
  int block_size;
  int kv_dtype;         /* etc_kv_dtype; must match the pool */
  int exact;            /* 1: reference-order arithmetic where it is cheap (f64 attention/norm/rope,
                           sequential-k dense linears); 0: fast tensor-core paths */
} etc_decoder_config;

typedef enum etc_weight_slot {
  ETC_W_TOK_EMBD = 0, ETC_W_ATTN_NORM = 1, ETC_W_Q = 2, ETC_W_K = 3, ETC_W_V = 4, ETC_W_O = 5,
  ETC_W_FFN_NORM = 6, ETC_W_GATE = 7, ETC_W_UP = 8, ETC_W_DOWN = 9, ETC_W_OUT_NORM = 10, ETC_W_HEAD = 11
} etc_weight_slot;

/* ---- GGUF v3 files (crates/runtime/src/gguf.rs; napi loadGguf / inspectGguf, native-addon.ts:316-325) ----
 * etc_gguf_open parses header, metadata table and tensor catalog (parse_gguf, gguf.rs:682-946) with the reference's
 * resource limits, overflow checks and message texts, reading no payload. Differences: GGML type codes 2 (Q4_0) and
 * 8 (Q8_0) are accepted as well, their least-major dimension must be divisible by 32 instead of 256.
 * Errors: malformed file -> ETC_INVALID_ARGUMENT "gguf: ..."; I/O -> ETC_TRANSFER "gguf: I/O failed: ...";
 * cancellation flag set -> ETC_CANCELLED "gguf: operation aborted". Strings returned live as long as the handle. */
typedef struct etc_gguf etc_gguf;
ETC_API etc_status etc_gguf_open(const char* path, const volatile int* cancelled, etc_gguf** out);
ETC_API etc_status etc_gguf_close(etc_gguf* file);
ETC_API etc_status etc_gguf_summary(const etc_gguf* file, const char** architecture, int64_t* metadata_count,
                                    int64_t* tensor_count);
/* One metadata entry in file order. value_type is the GGUF type code (9 = array, then element_type and count are set
 * and the scalar outputs hold the first element). Integers and bool come in integer_bits (two's complement for the
 * signed types), f32/f64 in real, strings in string. */
ETC_API etc_status etc_gguf_metadata(const etc_gguf* file, int64_t index, const char** key, int* value_type,
                                     int* element_type, int64_t* count, uint64_t* integer_bits, double* real,
                                     const char** string);
/* One catalog entry (GgufTensorDescriptor, gguf.rs:309-337): logical shape row-major (GGUF dimensions reversed);
 * physical shape = logical for F32, [rows, encoded_row_bytes] for block codecs; absolute, validated byte range. */
ETC_API etc_status etc_gguf_tensor(const etc_gguf* file, int64_t index, const char** name, etc_codec* codec, int* rank,
                                   int64_t* logical_shape4, int64_t* physical_shape4, uint64_t* data_offset,
                                   uint64_t* byte_len);
ETC_API etc_status etc_gguf_find_tensor(const etc_gguf* file, const char* name, int64_t* index);
/* read_gguf_tensor_into (gguf.rs:948-990): dst_bytes must equal the tensor's byte length exactly; positioned reads in
 * 8 MiB chunks with the cancellation flag polled between them. */
ETC_API etc_status etc_gguf_read_tensor_into(const etc_gguf* file, int64_t index, void* h_dst, uint64_t dst_bytes,
                                             const volatile int* cancelled);
/* The same payload streamed into device memory through two pinned staging buffers (file read of one chunk overlaps
 * the copy of the previous one); returns after the runtime's stream has the whole tensor. */
ETC_API etc_status etc_gguf_load_tensor_device(etc_runtime* rt, const etc_gguf* file, int64_t index, void* d_dst,
                                               uint64_t dst_bytes, const volatile int* cancelled);

/* Tensor parallelism (one process per GPU; no counterpart in the single-device reference). Each rank creates its
 * decoder with LOCAL geometry (q_heads/world, kv_heads/world, ffn/world; d_model whole; vocab whole unless the head is
 * sharded, see etc_decoder_set_head_shard) and binds its shard
 * of every projection: a contiguous row range of wq/wk/wv/gate/up, a contiguous range of 32-value blocks of every row
 * of wo/down; embedding, norms and head are replicated, and so is the host-side page allocation, so every rank's KV
 * pool (built with the local kv_heads) holds the same page tables. Rank 0 makes the 128-byte id, the host sends it to
 * every rank by its own means, and all ranks call etc_decoder_set_tensor_parallel together (it blocks until the last
 * one joins). After o and down the partial sums are all-reduced (f32, NCCL, on the runtime's stream, inside the
 * captured step graph as well); rank 0 alone adds the residual. world == 1 is accepted and changes nothing. */
ETC_API etc_status etc_tp_unique_id(uint8_t* out_id_128_bytes);
ETC_API etc_status etc_decoder_set_tensor_parallel(etc_decoder* dec, int rank, int world, const uint8_t* id_128_bytes);
/* Optional, after etc_decoder_set_tensor_parallel and etc_decoder_finalize: replace the NCCL all-reduce by the
 * library's kernel over peer memory (CUDA IPC, plain stores into the peers' regions over NVLink, 2..8 ranks on one
 * node): one shot up to 4 ranks (every rank receives all ranks' partial sums), reduce-scatter + all-gather at 8; the
 * row-parallel projection's split-K partials are summed inside the same kernel. Every rank exports a
 * 64-byte handle of its exchange region, the host gathers the handles of all ranks into a table [world][64] (own slot
 * ignored) and every rank imports it. The kernel's wait for its peers is bounded: a rank that never arrives turns
 * into ETC_EXECUTION at the next synchronising call, not into a hang. ETC_TP_TWO_SHOT=0 or 1 in the environment of the
 * importing call forces the one-shot or the reduce-scatter + all-gather form (every rank must use the same);
 * ETC_TP_CHAIN=0, 1 or 2 picks how the exchange kernel is launched relative to its neighbours (1, the default: after
 * the projection has ended, releasing its successor early), a knob for measurements only.
 * Two duties stay with the host, because a rank only sees its own status. (1) After every step the ranks exchange
 * their step status over the host transport; when any rank failed, every rank treats the step as failed (a rank whose
 * own call returned ETC_OK has committed already: it releases the affected sequences and re-creates them, as it would
 * after any other lost step). (2) Before a decoder is destroyed, or its peers re-imported, all ranks pass a host
 * barrier: a peer may still be reading this rank's exchange region until its own step has been synchronised. */
ETC_API etc_status etc_decoder_tp_peer_export(etc_decoder* dec, uint8_t* out_handle_64_bytes);
ETC_API etc_status etc_decoder_tp_peer_import(etc_decoder* dec, const uint8_t* handles_world_x_64_bytes);
/* The same without CUDA IPC, for hosts that map the peers' regions themselves (a virtual-memory mapping, or one process
 * that drives several devices): etc_decoder_tp_region returns this rank's region (allocated on first use, zeroed) and
 * its size; etc_decoder_tp_peer_attach takes every rank's region as a device pointer valid in this process (own slot
 * ignored). With these, etc_decoder_set_tensor_parallel may be called with a null id: no NCCL communicator is made and
 * the decoder steps only once the regions are attached. */
ETC_API etc_status etc_decoder_tp_region(etc_decoder* dec, void** out_region, size_t* out_bytes);
ETC_API etc_status etc_decoder_tp_peer_attach(etc_decoder* dec, void* const* regions_world);
/* Bound of every wait for a peer inside the decoder's kernels, in SM clock cycles (<= 0: the default, about a second).
 * A step whose wait runs out returns ETC_EXECUTION and is rolled back like any other failed step. */
ETC_API etc_status etc_decoder_set_wait_limit(etc_decoder* dec, int64_t cycles);
/* Vocabulary-parallel head, before any weight is bound: the decoder's config.vocab is the number of head rows this rank
 * holds, rows [first_row, first_row + config.vocab) of a head with `vocab_global` rows; the token embedding keeps
 * vocab_global rows on every rank. Greedy steps then exchange every rank's (best logit, token) pair over the peer
 * regions (etc_decoder_tp_peer_import is required) and keep the largest logit, on ties the lowest token, exactly what
 * an ascending scan with a strict comparison finds on one device (crates/runtime/src/sampling.rs:88-105).
 * etc_decoder_execute returns this rank's [active, config.vocab] slice of the logits. */
ETC_API etc_status etc_decoder_set_head_shard(etc_decoder* dec, int64_t vocab_global, int64_t first_row);
/* The peer-memory all-reduce as an operator of its own. A region is etc_peer_region_bytes(capacity, world) bytes of
 * device memory, zeroed once before its first use; regions[r] is rank r's region as mapped in this process (own rank:
 * local memory). hidden[0, count) += sum over ranks of their partial sums (d_partial is this rank's): every rank stores
 * its partial sum (two_shot: slice q of it to rank q) into the peers' regions, buffer `buffer` (0 or 1, alternating
 * between consecutive calls), and adds up what the peers stored into its own. count is a multiple of 4, at most
 * `capacity`. wait_cycles bounds the wait for the peers in SM clock cycles (<= 0: about one second); when it runs out
 * the launch gives up and the next synchronising call returns ETC_EXECUTION, the runtime stays usable. */
ETC_API size_t etc_peer_region_bytes(int64_t capacity, int world);
ETC_API etc_status etc_peer_allreduce_into(etc_runtime* rt, int rank, int world, void* const* regions, int64_t capacity,
                                           int buffer, const float* d_partial, float* d_hidden, int64_t count, int two_shot,
                                           int64_t wait_cycles);

/* The attention half of kv_attention_into alone, over lane descriptors and block tables that already sit in device
 * memory (the decode kernel of napi/mod.rs:3478-3540 for one query token per lane; what the Metal backend's paged kernel
 * takes as block_tables / context lengths / block_bases, crates/runtime-metal/src/paged.rs:651-795). Asynchronous and
 * free of host state: nothing is allocated, no page is drawn, no cursor moves, so the call can be captured into a CUDA
 * graph and replayed. d_lanes[i] = {cursor, advance (1 = live lane, 0 = padded), start (first resident position),
 * table_offset (index in d_tables of the block that holds position 0)}; lane i attends over positions [start, cursor +
 * advance) (further narrowed by op_window). max_pages bounds the pages any lane attends over and fixes the split plan;
 * d_scratch holds etc_kv_attention_plan(...).partial_bytes for that plan. Needs an f16 / bf16 pool with 16-token pages. */
typedef struct etc_lane { int cursor, advance, start, table_offset; } etc_lane;
ETC_API etc_status etc_paged_attention_into(etc_runtime* rt, etc_pool* pool, int layer, const etc_lane* d_lanes,
                                            const int* d_tables, int batch, int max_pages, const float* d_q, int q_heads,
                                            double scale, int64_t op_window, float* d_out, void* d_scratch,
                                            size_t scratch_bytes);

/* Planners of the flash-decoding kernel, pure host arithmetic in the manner of the reference's `*_requirements`
 * calls (crates/runtime-cpu/src/lib.rs:5-11). etc_kv_attention_plan: the split of `attended_pages` pages over the grid
 * and the bytes of split partials one launch writes. etc_decoder_attention_reserve: the longest block table a decoder of
 * this configuration stages per lane and the partial bytes it sets aside at finalize; every plan a step can ask for
 * (any table length up to max_blocks, rounded up to 8 pages as captured steps do) fits in it. */
ETC_API etc_status etc_kv_attention_plan(int batch, int q_heads, int kv_heads, int head_dim, int attended_pages, int sm_count,
                                         int* splits, int* pages_per_split, size_t* partial_bytes);
ETC_API etc_status etc_decoder_attention_reserve(const etc_decoder_config* config, int max_advance, int sm_count,
                                                 int* max_blocks, size_t* partial_bytes);

ETC_API etc_status etc_decoder_create(etc_runtime* rt, const etc_decoder_config* config, etc_decoder** out);
ETC_API etc_status etc_decoder_destroy(etc_decoder* dec);
/* Bind one weight (host pointer; uploaded and retained — constantWeights). codec F32 = dense f32
 * [rows, columns] (norm vectors: rows = 1); otherwise raw packed GGUF rows. */
ETC_API etc_status etc_decoder_set_weight(etc_decoder* dec, etc_weight_slot slot, int layer, etc_codec codec,
                                          const void* h_data, int64_t rows, int64_t columns);
/* Same, from device memory already holding the raw tensor. */
ETC_API etc_status etc_decoder_set_weight_device(etc_decoder* dec, etc_weight_slot slot, int layer, etc_codec codec,
                                                 const void* d_data, int64_t rows, int64_t columns);
/* Longest chunk (tokens per sequence per call) the decoder will be asked to run; default 1. The
 * reference compiles one program per chunk shape ([1,prefillChunk], [1,1], [batch,1],
 * packages/core/src/Model.ts:1906-1946); here one decoder serves every advance up to this bound. */
ETC_API etc_status etc_decoder_set_max_advance(etc_decoder* dec, int max_advance);
/* Freeze the plan: fuse q/k/v and gate/up matrices, size workspaces. */
ETC_API etc_status etc_decoder_finalize(etc_decoder* dec);

/* Executable.execute for a stateful program: `active` sequences (1..=batch) each advance by
 * `advance` tokens (h_tokens is [active, advance] u32); h_logits (may be NULL) receives the
 * LastTokenRow logits [active, vocab]. Pads to the compiled batch, runs begin -> commands ->
 * commit; any failure (pool exhausted, capacity, cancellation, device status) rolls back so no
 * cursor or block list changes (napi/mod.rs:4441-4518). `cancelled` may be NULL. */
ETC_API etc_status etc_decoder_execute(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active,
                                       const uint32_t* h_tokens, int advance, float* h_logits,
                                       const volatile int* cancelled);
/* Executable.executeSampled with greedy sampling before commit: h_out_tokens [active]. */
ETC_API etc_status etc_decoder_execute_sampled(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active,
                                               const uint32_t* h_tokens, int advance, uint32_t* h_out_tokens,
                                               const volatile int* cancelled);
/* Device-resident variant for benchmarking the kernel schedule alone: runs `steps` greedy decode
 * steps back to back feeding each step's tokens to the next, without host round trips in between;
 * h_out_tokens [steps, active]. Commits every step. */
ETC_API etc_status etc_decoder_generate_greedy(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active,
                                               const uint32_t* h_first_tokens, int steps, uint32_t* h_out_tokens,
                                               float* out_device_ms);
/* Kernels launched per decode step by the current plan, and per-kernel-class device time of the
 * last profiled step (ExecutableDiagnostics analogue, crates/runtime/src/executable.rs:26-35). */
ETC_API etc_status etc_decoder_diagnostics(etc_decoder* dec, int* launches_per_step, uint64_t* weight_bytes,
                                           uint64_t* workspace_bytes);

#ifdef __cplusplus
}
#endif
#endif /* ET_CUDA_H */
