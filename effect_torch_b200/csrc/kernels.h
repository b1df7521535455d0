// Host-callable launchers of the CUDA kernels (implemented in the .cu files). All launch on the
// given stream and return the cudaError_t of the launch. Pointers are device pointers.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "common.h"

namespace etc {

// ---- block-quantized weights (quant_kernels.cu) ------------------------------------------
cudaError_t launch_dequantize(int codec, const uint8_t* packed, int64_t rows, int64_t columns, float* out,
                              cudaStream_t stream);
cudaError_t launch_quantize(int codec, const float* x, int64_t rows, int64_t columns, uint8_t* packed,
                            cudaStream_t stream);
cudaError_t launch_qlinear_generic(int codec, const float* x, int64_t vectors, int64_t columns, const uint8_t* weight,
                                   int64_t rows, const float* bias, float* out, cudaStream_t stream, int* launches);
cudaError_t launch_qembedding(int codec, const void* indexes, int index_is_i64, int64_t count, const uint8_t* weight,
                              int64_t rows, int64_t columns, float* out, DeviceStatus* status, cudaStream_t stream);

// Tiled weights (Q4_0 / Q8_0): 128-row tiles. For row tile t and 32-column block kb the 128 rows' 16 (Q4_0) or 32
// (Q8_0) payload bytes are contiguous ([tile][block][row][bytes]; Q4_0 nibbles pre-ordered so that masks give f16 pairs
// in column order), scales are [tile][block][row] f16. Same byte count as the GGUF encoding; rows padded to 128 with
// zero scales. Both linear kernels (qlinear_mv.cu, qlinear_umma.cu) read this one layout.
// A run of 128-row tiles of one codec inside a tiled weight. A weight fused from parts of different codecs (q and k in
// Q4_K, v in Q6_K, as GGUF files mix them) holds one segment per run of equal codecs, each repacked in its codec's layout
// at byte offsets into the weight's arrays; the linear launches one kernel per segment into the same outputs.
struct TiledSegment {
  int codec = 0;
  int tile0 = 0, tiles = 0;
  size_t quant_offset = 0, scale_offset = 0;  // bytes
};
constexpr int kMaxSegments = 4;

struct TiledWeight {
  int codec = 0;            // the first segment's codec
  int64_t rows = 0;         // logical rows (outputs) after concatenation / interleave
  int64_t rows_padded = 0;  // multiple of 128
  int64_t columns = 0;      // multiple of 64
  int interleave8 = 0;
  uint8_t* quants = nullptr;
  __half* scales = nullptr;
  size_t quant_bytes = 0, scale_bytes = 0;
  // [rows_padded/128] arrival tickets, zero between launches: taken by the matvec kernel's CTAs that hold part of a row
  // group's K; the last one to arrive finishes the group
  int* counters = nullptr;
  int n_segments = 0;       // 0: one segment of `codec` over the whole weight
  TiledSegment segments[kMaxSegments];
};
// Split-K partials a linear left unsummed for the kernel that consumes its result (the next RMSNorm, or the RoPE /
// KV-append kernel): [splits][vpad][rows_padded] f32, summed in split order. splits == 0: the result is already in `out`.
struct DeferredSum {
  const float* partials = nullptr;
  int splits = 0, vpad = 0, rows_padded = 0;
};

struct RepackParts {
  const uint8_t* ptr[4];
  int64_t rows[4];
  int n_parts;
};
cudaError_t launch_repack(const TiledWeight& w, const RepackParts& parts, cudaStream_t stream);

// out_xh (optional): the result also stored as f16 in [cols/8][xh_nv][8] order for the next linear.
cudaError_t launch_qlinear_reduce(const float* scratch, int splits, int vpad, int vectors, int rows, int rows_padded,
                                  const float* bias, const float* residual, int epilogue, float* out, __half* out_xh,
                                  cudaStream_t stream, int xh_nv = 32);

// tcgen05 path (qlinear_umma.cu)
struct UmmaPlan {
  int nv = 32;               // vectors per chunk padded to the MMA N (32, 64, 128 or 256)
  int chunks = 1;            // chunks of nv vectors the call is cut into (grid.z); more than one only at nv = 256
  int tiles = 1, splits = 1, blocks_per_split = 0;
  size_t xh_bytes = 0;       // f16 activations in [chunk][K/8][nv][8] order, all chunks
  size_t scratch_bytes = 0;  // split-K partials [chunk][split][nv][rows_padded], all chunks
};
UmmaPlan plan_umma(const TiledWeight& w, int64_t vectors, int sm_count);
cudaError_t launch_repack_umma(const TiledWeight& w, const RepackParts& parts, cudaStream_t stream);
// x: f32 [vectors, K], converted to xh8 into `xh` first — unless xh_ready (already [K/8][32][8] f16, vectors <= 32) is given.
cudaError_t launch_qlinear_umma(const TiledWeight& w, const float* x, const __half* xh_ready, int64_t vectors, const float* bias,
                                const float* residual, int epilogue, float* out, __half* out_xh, __half* xh, float* scratch,
                                DeviceStatus* status, int sm_count, cudaStream_t stream, int* launches, int xh_nv = 32,
                                DeferredSum* defer = nullptr);

// small-batch matvec on the 128-row layout (qlinear_mv.cu): up to 32 vectors per pass, mma.sync fed by a bulk-copy ring
struct MvPlan {
  int nt = 1;  // groups of 8 vectors per pass (1, 2 or 4)
  int tiles = 1, groups = 1, spt = 1, units = 1, upc = 1, grid = 1;  // row groups of 1-2 tiles, stages per group, (group, stage) units, units per CTA
  size_t xh_bytes = 0;       // f16 activations [K/8][nt*8][8] when the caller passes f32 rows (rounded to 256 bytes)
  size_t partial_bytes = 0;  // [grid][2][nt*8][128] f32 partial tiles of runs that cover part of a tile's K
};
MvPlan plan_mv(const TiledWeight& w, int64_t vectors, int sm_count);
// Largest vector count the front end routes to the matvec kernel (the tcgen05 kernel takes over above it).
int mv_max_vectors();
// x f32 [vectors, K] (converted into the head of `scratch` first), or xh_ready in the f16 hand-off layout with row stride
// xh_nv; scratch holds xh_bytes + partial_bytes of the plan; w.counters holds the tile tickets.
cudaError_t launch_qlinear_mv(const TiledWeight& w, const float* x, const __half* xh_ready, int64_t vectors, const float* bias,
                              const float* residual, int epilogue, float* out, __half* out_xh, void* scratch,
                              DeviceStatus* status, int sm_count, cudaStream_t stream, int* launches, int xh_nv = 32);

// Front end of the tiled linear. `scratch` must hold tiled_scratch_bytes(w, vectors, sm_count).
size_t tiled_scratch_bytes(const TiledWeight& w, int64_t vectors, int sm_count);
// xh_ready / out_xh: optional f16 activation hand-off between kernels, [K/8][xh_nv][8] with xh_nv = hand_off_stride(batch)
// (up to 128 vectors).
cudaError_t launch_qlinear_tiled(const TiledWeight& w, const float* x, int64_t vectors, const float* bias,
                                 const float* residual, int epilogue, float* out, void* scratch, DeviceStatus* status,
                                 int sm_count, cudaStream_t stream, int* launches, const __half* xh_ready = nullptr,
                                 __half* out_xh = nullptr, int xh_nv = 32, DeferredSum* defer = nullptr);
// Row stride of the f16 hand-off layout for `vectors` rows: 32, 64 or 128 (0: no hand-off above 128 vectors).
inline int hand_off_stride(int64_t vectors) { return vectors <= 32 ? 32 : (vectors <= 64 ? 64 : (vectors <= 128 ? 128 : 0)); }
// RMSNorm whose output is stored as f16 [n/8][xh_nv][8] (rows <= xh_nv).
cudaError_t launch_rmsnorm_xh8(const float* x, const float* weight, double eps, int64_t rows, int64_t n, __half* out_xh,
                               cudaStream_t stream, int xh_nv = 32);
// The same after x += sum of a projection's split-K partials (x is updated in place: the residual stream).
cudaError_t launch_sum_rmsnorm_xh8(float* x, const DeferredSum& sum, const float* weight, double eps, int64_t rows, int64_t n,
                                   __half* out_xh, cudaStream_t stream, int xh_nv = 32);

// ---- tensor-parallel all-reduce over peer memory (tp_kernels.cu) -----------------------------
constexpr int kMaxTpRanks = 8;
// One rank's exchange region: [0, 96) three flag arrays of kTpFlagStride words (partial sums stored, slice totals stored,
// picks stored), [256, 288) counters private to the owner, [1024, 1024 + 8 * kTpMaxPicks) (best logit, token) pairs, then
// from kTpHeaderBytes on two exchange buffers of (world + 1) slots of `slot_bytes` each: an inbox with one slot per
// sender, and the table of totals.
constexpr int kTpFlagStride = 8;
constexpr size_t kTpCounterOffset = 256, kTpPickOffset = 1024, kTpHeaderBytes = 4096;
constexpr int kTpMaxPicks = 256;
constexpr long long kTpWaitCycles = 1ll << 31;  // about a second
struct PeerView {
  float* inbox[kMaxTpRanks][2];   // every rank's inboxes [world][slot] (own: local memory, others: peer mappings)
  float* totals[kMaxTpRanks][2];  // every rank's tables of slice totals [slot]
  uint32_t* flags[kMaxTpRanks];   // every rank's flag arrays; entry r of each is written by rank r
  uint2* picks[kMaxTpRanks];      // every rank's (best logit bits, token) per lane
  int rank, world;
};
inline size_t tp_slot_bytes(size_t capacity_floats) { return (capacity_floats * sizeof(float) + 255) & ~(size_t)255; }
inline size_t tp_region_bytes(size_t capacity_floats, int world) {
  return kTpHeaderBytes + 2 * (size_t)(world + 1) * tp_slot_bytes(capacity_floats);
}
inline void tp_view_bind(PeerView& view, int r, unsigned char* base, size_t slot_bytes, int world) {
  view.flags[r] = reinterpret_cast<uint32_t*>(base);
  view.picks[r] = reinterpret_cast<uint2*>(base + kTpPickOffset);
  for (int b = 0; b < 2; ++b) {
    unsigned char* buffer = base + kTpHeaderBytes + (size_t)b * (world + 1) * slot_bytes;
    view.inbox[r][b] = reinterpret_cast<float*>(buffer);
    view.totals[r][b] = reinterpret_cast<float*>(buffer + (size_t)world * slot_bytes);
  }
}
// hidden[0, count) += sum over ranks of their partial sums; count is a multiple of 4. This rank's partial sum is
// `partial`, or with sum.splits > 0 the sum of the split-K partials of a [count / columns, columns] projection result.
cudaError_t launch_tp_allreduce(const PeerView& view, int buffer, float* hidden, size_t count, int columns, const DeferredSum& sum,
                                const float* partial, bool two_shot, uint32_t* counters, long long wait_cycles, int sm_count,
                                DeviceStatus* status, cudaStream_t stream);
// tokens[b] = the token of the largest logit over all ranks' picks (lowest token on ties), b < batch <= kTpMaxPicks.
cudaError_t launch_tp_pick(const PeerView& view, int batch, uint32_t* tokens, uint32_t* counters, long long wait_cycles,
                           DeviceStatus* status, cudaStream_t stream);

// ---- dense / elementwise (elementwise.cu) --------------------------------------------------
cudaError_t launch_linear_f32(const float* x, int64_t m, int64_t k, const float* w, int64_t n, const float* bias,
                              float* out, cudaStream_t stream);
cudaError_t launch_rmsnorm(const float* x, const float* weight, double eps, int64_t rows, int64_t n, float* out,
                           cudaStream_t stream);
cudaError_t launch_rope(const float* x, const int64_t* offsets, int64_t n_offsets, const double* inv_freq, int layout,
                        int64_t batch, int64_t heads, int64_t steps, int64_t head_dim, float* out, cudaStream_t stream);
cudaError_t launch_swiglu(const float* gate, const float* up, int64_t n, float* out, int exact, cudaStream_t stream);
cudaError_t launch_add(const float* a, const float* b, int64_t n, float* out, cudaStream_t stream);
cudaError_t launch_argmax(const float* logits, int64_t rows, int64_t vocab, uint32_t* tokens, DeviceStatus* status,
                          cudaStream_t stream,
                          uint2* picks = nullptr, uint32_t index_base = 0);
// One token per logits row by temperature / top-k / top-p sampling with the splitmix64 draw (sampling.cu); temperature
// must be positive here (zero is the argmax kernel's case). seeds / counters: optional per-row device arrays.
cudaError_t launch_sample_rows(const float* logits, int64_t rows, int64_t vocab, double temperature, int64_t top_k, double top_p,
                               uint64_t seed, uint64_t counter, const uint64_t* seeds, const uint64_t* counters, uint32_t* tokens,
                               DeviceStatus* status, cudaStream_t stream);
cudaError_t launch_embedding_f32(const void* indexes, int index_is_i64, int64_t count, const float* table, int64_t rows,
                                 int64_t columns, float* out, DeviceStatus* status, cudaStream_t stream);
// [B,T,H*D] <-> [B,H,T,D] (the reshape/transpose pairs around attention)
cudaError_t launch_heads_first(const float* src, float* dst, int64_t B, int64_t T, int64_t H, int64_t D, int64_t src_row_stride,
                               cudaStream_t stream);
cudaError_t launch_heads_last(const float* src, float* dst, int64_t B, int64_t T, int64_t H, int64_t D,
                              cudaStream_t stream);
// Copy row (advance-1) of each lane's [T, width] block into [lanes, width] (LastTokenRow).
cudaError_t launch_last_token_rows(const float* src, int64_t lanes, int64_t steps, int64_t width, int64_t advance,
                                   float* out, cudaStream_t stream);

// ---- paged KV (attention.cu) -----------------------------------------------------------------
// Device pool geometry. Page-major layout chosen for the B200: each (page, kv head) holds its
// block_size token rows contiguously: elem(page, head, slot, d) = ((page*kv_heads + head)*block_size + slot)*head_dim + d.
struct PoolView {
  void* k = nullptr;       // this layer's K slab
  void* v = nullptr;
  float* k_scale = nullptr;  // u8 tier: [page][head][slot]
  float* v_scale = nullptr;
  int dtype = 0, kv_heads = 0, head_dim = 0, block_size = 0;
};
// Per-lane step description in device memory.
struct LaneInfo {
  int cursor;      // tokens already committed
  int advance;     // live query rows in this step (0 = padded lane)
  int start;       // first position still resident (pool window), 0 without
  int table_offset;  // offset of this lane's block table in the tables array (index 0 = block of position 0)
};
cudaError_t launch_kv_append(const PoolView& pool, const float* k, const float* v, const LaneInfo* lanes,
                             const int* tables, int batch, int tokens, int64_t lane_stride, int64_t head_stride,
                             int64_t token_stride, cudaStream_t stream);
// Reference-order attention in f64 (any tier, any block size, window). q/out [B,Hq,T,D] f32.
// scratch: f64 [B*Hq*T][max_ctx]. op_window < 0: none.
cudaError_t launch_attention_exact(const PoolView& pool, const float* q, const LaneInfo* lanes, const int* tables,
                                   int batch, int q_heads, int tokens, double scale, long long op_window, float* out,
                                   double* scratch, int max_ctx, cudaStream_t stream);
// Tensor-core flash-decoding over the block table (f16/bf16 tiers, block_size 16, head_dim 64/128,
// one query token per lane). q [B,Hq,D] f32; out [B,Hq,D] f32. partial scratch for splits > 1.
struct AttnPlan {
  int splits = 1;
  int pages_per_split = 0;
  size_t scratch_bytes = 0;
};
AttnPlan plan_attention(int batch, int q_heads, int kv_heads, int head_dim, int max_pages, int sm_count);
// Largest scratch plan_attention can ask for with tables of at most max_pages pages.
size_t plan_attention_max_scratch(int batch, int q_heads, int kv_heads, int head_dim, int max_pages, int sm_count);
bool attention_mma_supported(const PoolView& pool, int q_heads, int tokens);
cudaError_t launch_attention_mma(const PoolView& pool, const float* q, const LaneInfo* lanes, const int* tables,
                                 int batch, int q_heads, double scale, long long op_window, float* out,
                                 const AttnPlan& plan, float* scratch, cudaStream_t stream, int* launches,
                                 __half* out_xh = nullptr, int xh_nv = 32, int tokens = 1);
// Fused RoPE(q), RoPE(k) and KV append: qkv [B * tokens, (Hq+2*Hkv)*D] f32 (the fused projection output) ->
// q_out [B, tokens, Hq, D] f32 rotated, K/V rows written to the pool at positions cursor .. cursor + tokens - 1.
cudaError_t launch_rope_append(const PoolView& pool, const float* qkv, const LaneInfo* lanes, const int* tables,
                               const double* inv_freq, int layout, int batch, int q_heads, float* q_out,
                               cudaStream_t stream, const DeferredSum* sum = nullptr, int tokens = 1);
// Tail of a device-resident greedy step: feeds the sampled tokens back as the next ids, appends
// them to the history, and advances every live lane's cursor (and window start) by one.
cudaError_t launch_record_step(const uint32_t* tokens, uint32_t* ids, uint32_t* history, int* step_counter, LaneInfo* lanes,
                               int64_t* cursors, int batch, long long window, cudaStream_t stream);
cudaError_t launch_pool_read_rows(const PoolView& pool, const uint32_t* rows, int64_t n, float* out, int which,
                                  cudaStream_t stream);

}  // namespace etc
