// Paged KV kernels for sm_100a: page-pool append (all four tiers), reference-order attention in
// f64, tensor-core flash-decoding over the block table with split-KV merge, and the fused
// RoPE + append used by one-token decode steps.
//
// Replaces kv_attention_into of the reference (crates/runtime-cpu/src/napi/mod.rs:3320-3565):
// the scatter (:3397-3459) and the attend loop (:3461-3542), and the slab tiers of
// crates/runtime-cpu/src/pool.rs:20-257.
//
// HBM layout (chosen for the B200, not the reference's token-major slab): per layer one K and
// one V slab of [pages][kv_heads][block_size][head_dim] elements, so the block_size rows of one
// (page, head) are one contiguous run (4 KiB for f16, 16 tokens, D=128) that a warp fetches
// with 16-byte cp.async copies. u8 tier scales are [pages][kv_heads][block_size] f32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "chain.cuh"
#include "kernels.h"

namespace etc {

enum : int { kKvF32 = 0, kKvF16 = 1, kKvBF16 = 2, kKvU8 = 3 };

__device__ __forceinline__ size_t pool_elem(const PoolView& p, int page, int head, int slot) {
  return (((size_t)page * p.kv_heads + head) * p.block_size + slot) * p.head_dim;
}
__device__ __forceinline__ size_t pool_scale_index(const PoolView& p, int page, int head, int slot) {
  return ((size_t)page * p.kv_heads + head) * p.block_size + slot;
}

// Widening read of one cached element (pool.rs:51-58; the u8 tier applies (code-128)*scale as
// napi/mod.rs:3474-3476 does).
__device__ __forceinline__ float pool_load(const PoolView& p, const void* slab, const float* scales, size_t elem,
                                           size_t scale_index) {
  switch (p.dtype) {
    case kKvF32: return reinterpret_cast<const float*>(slab)[elem];
    case kKvF16: return __half2float(reinterpret_cast<const __half*>(slab)[elem]);
    case kKvBF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(slab)[elem]);
    default: return __fmul_rn(__fsub_rn((float)reinterpret_cast<const uint8_t*>(slab)[elem], 128.0f), scales[scale_index]);
  }
}

// --------------------------------------------------------------------------------------------
// KV append: grid (tokens, kv_heads, batch), one CTA per (lane, head, new token) row.
// k/v are f32 with explicit strides so both the reference layout [B,Hkv,T,D] and the fused
// projection output [B, ...] can be scattered. u8 tier: scale = absmax/127 + 1e-12,
// code = clamp(round(x/scale), +-127) + 128 with round = ties away from zero (pool.rs:224-240).
// --------------------------------------------------------------------------------------------
__global__ void kv_append_kernel(PoolView pool, const float* __restrict__ k, const float* __restrict__ v,
                                 const LaneInfo* __restrict__ lanes, const int* __restrict__ tables, int64_t lane_stride,
                                 int64_t head_stride, int64_t token_stride) {
  __shared__ float red[2][32];
  const int token = blockIdx.x, head = blockIdx.y, lane_id = blockIdx.z;
  const LaneInfo info = lanes[lane_id];
  if (token >= info.advance) return;  // padded lane or dead row of the chunk
  const int pos = info.cursor + token;
  const int page = tables[info.table_offset + pos / pool.block_size];
  const int slot = pos % pool.block_size;
  const size_t dst = pool_elem(pool, page, head, slot);
  const float* ksrc = k + lane_id * lane_stride + head * head_stride + token * token_stride;
  const float* vsrc = v + lane_id * lane_stride + head * head_stride + token * token_stride;
  const int D = pool.head_dim;
  if (pool.dtype == kKvU8) {
    float kmax = 0.0f, vmax = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      kmax = fmaxf(kmax, fabsf(ksrc[d]));
      vmax = fmaxf(vmax, fabsf(vsrc[d]));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      kmax = fmaxf(kmax, __shfl_xor_sync(0xffffffffu, kmax, off));
      vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
    }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = kmax; red[1][threadIdx.x >> 5] = vmax; }
    __syncthreads();
    kmax = 0.0f; vmax = 0.0f;
    for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) { kmax = fmaxf(kmax, red[0][w]); vmax = fmaxf(vmax, red[1][w]); }
    const float kscale = __fadd_rn(__fdiv_rn(kmax, 127.0f), 1e-12f);
    const float vscale = __fadd_rn(__fdiv_rn(vmax, 127.0f), 1e-12f);
    if (threadIdx.x == 0) {
      const size_t si = pool_scale_index(pool, page, head, slot);
      pool.k_scale[si] = kscale;
      pool.v_scale[si] = vscale;
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float kc = roundf(__fdiv_rn(ksrc[d], kscale));
      float vc = roundf(__fdiv_rn(vsrc[d], vscale));
      kc = fminf(fmaxf(kc, -127.0f), 127.0f) + 128.0f;
      vc = fminf(fmaxf(vc, -127.0f), 127.0f) + 128.0f;
      reinterpret_cast<uint8_t*>(pool.k)[dst + d] = (uint8_t)kc;
      reinterpret_cast<uint8_t*>(pool.v)[dst + d] = (uint8_t)vc;
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float kv = ksrc[d], vv = vsrc[d];
    if (pool.dtype == kKvF32) {
      reinterpret_cast<float*>(pool.k)[dst + d] = kv;
      reinterpret_cast<float*>(pool.v)[dst + d] = vv;
    } else if (pool.dtype == kKvF16) {
      reinterpret_cast<__half*>(pool.k)[dst + d] = __float2half_rn(kv);
      reinterpret_cast<__half*>(pool.v)[dst + d] = __float2half_rn(vv);
    } else {
      reinterpret_cast<__nv_bfloat16*>(pool.k)[dst + d] = __float2bfloat16_rn(kv);
      reinterpret_cast<__nv_bfloat16*>(pool.v)[dst + d] = __float2bfloat16_rn(vv);
    }
  }
}

cudaError_t launch_kv_append(const PoolView& pool, const float* k, const float* v, const LaneInfo* lanes,
                             const int* tables, int batch, int tokens, int64_t lane_stride, int64_t head_stride,
                             int64_t token_stride, cudaStream_t stream) {
  if (batch == 0 || tokens == 0) return cudaSuccess;
  dim3 grid((unsigned)tokens, (unsigned)pool.kv_heads, (unsigned)batch);
  const int threads = std::min(128, ((pool.head_dim + 31) / 32) * 32);
  kv_append_kernel<<<grid, threads, 0, stream>>>(pool, k, v, lanes, tables, lane_stride, head_stride, token_stride);
  return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------
// Reference-order attention. One CTA per (query head, query row, lane). Scores are f64 dot
// products accumulated over the head dimension in index order (the products of two f32 values are
// exact in f64, so this equals the reference's sum bit for bit), scaled, max-reduced; the weights
// exp(s*scale - max) are kept in a global f64 scratch row; then thread c accumulates column c of
// the output over positions in order with separate multiply and add, exactly like the
// reference's loop, and divides by the denominator it accumulated the same way.
// Only exp() can differ from the host libm, by an ulp of f64.
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) attention_exact_kernel(PoolView pool, const float* __restrict__ q,
                                                              const LaneInfo* __restrict__ lanes,
                                                              const int* __restrict__ tables, int q_heads, int tokens,
                                                              double scale, long long op_window, float* __restrict__ out,
                                                              double* __restrict__ scratch, int max_ctx) {
  __shared__ double red[4];
  __shared__ double max_s;
  const int head = blockIdx.x, query = blockIdx.y, lane_id = blockIdx.z;
  const LaneInfo info = lanes[lane_id];
  const int D = pool.head_dim;
  const size_t row_index = ((size_t)lane_id * q_heads + head) * tokens + query;
  float* orow = out + row_index * D;
  if (info.advance == 0) {  // padded lane: output stays zero (napi/mod.rs:3371-3372)
    for (int d = threadIdx.x; d < D; d += blockDim.x) orow[d] = 0.0f;
    return;
  }
  const int kv_head = head / (q_heads / pool.kv_heads);
  const int needed = info.cursor + info.advance;
  const int end = min(info.cursor + query + 1, needed);
  int begin = info.start;
  if (op_window >= 0) begin = max((int)max((long long)end - op_window, 0ll), info.start);
  const int span = max(end - begin, 0);
  const float* qrow = q + row_index * D;
  double* wrow = scratch + row_index * (size_t)max_ctx;
  const int* table = tables + info.table_offset;

  double local_max = -INFINITY;
  for (int i = threadIdx.x; i < span; i += blockDim.x) {
    const int pos = begin + i;
    const int page = table[pos / pool.block_size], slot = pos % pool.block_size;
    const size_t base = pool_elem(pool, page, kv_head, slot);
    const size_t si = pool_scale_index(pool, page, kv_head, slot);
    double score = 0.0;
    for (int c = 0; c < D; ++c) score += (double)qrow[c] * (double)pool_load(pool, pool.k, pool.k_scale, base + c, si);
    const double scaled = __dmul_rn(score, scale);
    wrow[i] = scaled;
    local_max = fmax(local_max, scaled);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) local_max = fmax(local_max, __shfl_xor_sync(0xffffffffu, local_max, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local_max;
  __syncthreads();
  if (threadIdx.x == 0) {
    double m = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmax(m, red[w]);
    max_s = m;
  }
  __syncthreads();
  const double maximum = max_s;
  for (int i = threadIdx.x; i < span; i += blockDim.x) wrow[i] = exp(__dsub_rn(wrow[i], maximum));
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    double result = 0.0, denominator = 0.0;
    for (int i = 0; i < span; ++i) {
      const int pos = begin + i;
      const int page = table[pos / pool.block_size], slot = pos % pool.block_size;
      const double w = wrow[i];
      const float value = pool_load(pool, pool.v, pool.v_scale, pool_elem(pool, page, kv_head, slot) + c,
                                    pool_scale_index(pool, page, kv_head, slot));
      result = __dadd_rn(result, __dmul_rn(w, (double)value));
      denominator = __dadd_rn(denominator, w);
    }
    orow[c] = (float)__ddiv_rn(result, denominator);
  }
}

cudaError_t launch_attention_exact(const PoolView& pool, const float* q, const LaneInfo* lanes, const int* tables,
                                   int batch, int q_heads, int tokens, double scale, long long op_window, float* out,
                                   double* scratch, int max_ctx, cudaStream_t stream) {
  if (batch == 0 || tokens == 0) return cudaSuccess;
  dim3 grid((unsigned)q_heads, (unsigned)tokens, (unsigned)batch);
  attention_exact_kernel<<<grid, 128, 0, stream>>>(pool, q, lanes, tables, q_heads, tokens, scale, op_window, out,
                                                   scratch, max_ctx);
  return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------
// Tensor-core flash-decoding (one query token per lane, f16 or bf16 pages of 16 tokens).
//
// Grid (splits, kv_heads, batch); a CTA of 4 warps serves one (lane, kv head, page range) and all
// G = q_heads/kv_heads query heads of that KV head at once: the G query rows are rows 0..G-1 of
// the m16n8k16 A operand, so every K/V page is fetched from HBM once per KV head, not once per
// query head. Warps take pages round-robin; each warp keeps a 3-deep cp.async ring of
// (K page, V page) in shared memory (16-byte copies, XOR-swizzled so ldmatrix is conflict-free),
// computes S = Q K^T with mma.sync, the online softmax in registers (exp2 domain, scale*log2(e)
// folded into Q), P V with mma.sync reusing the S accumulators as the A operand, and at the end
// the 4 warps merge their (m, l, O) through shared memory. With splits > 1 the CTA writes an
// unnormalised partial (m, l, O) per query head and attention_merge_kernel combines the splits.
//
// Roofline: HBM-bound: bytes = sum_lanes ctx * 2 * kv_heads * D * sizeof(kv) (+ q, out, tables).
// --------------------------------------------------------------------------------------------
constexpr int kAttnWarps = 4;
constexpr int kAttnStages = 3;
constexpr int kPageTokens = 16;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct AttnArgs {
  const void* k;
  const void* v;
  const float* k_scale;    // u8 tier: one f32 per (page, head, slot)
  const float* v_scale;
  const float* q;          // [B, Hq, D] f32
  const LaneInfo* lanes;
  const int* tables;
  float* out;              // [B, Hq, D] f32 (splits == 1)
  __half* out_xh;          // optional f16 copy of out in [Hq*D/8][out_xh_nv][8] order: the o-projection's B operand
  int out_xh_nv;
  float* partial;          // [B, Hq, splits, D + 2] f32: O unnormalised, then m (log2 domain), l
  int q_heads, kv_heads;
  int pages_per_split;
  int tokens;              // query tokens per lane (1: decode; > 1: a prefill chunk, q and out are [B, tokens, Hq, D])
  float scale_log2;        // scale * log2(e)
  long long op_window;
};

// smem per warp per stage: K page then V page, each 16 rows x D*2 bytes, 16-byte chunk c of row r
// stored at chunk (c ^ (r & 7)) within its 128-byte group.
template <int D>
__device__ __forceinline__ int swizzled_offset(int row, int chunk) {  // in bytes
  return row * (D * 2) + ((chunk & ~7) | ((chunk ^ row) & 7)) * 16;
}

// CHUNK = false: one query token per lane; the 16 MMA rows are the query heads of one KV head and grid.x splits the pages.
// CHUNK = true: a chunk of a.tokens query tokens per lane (chunked prefill, napi/mod.rs:3420-3477 semantics: token t of
// the chunk attends positions up to cursor + t); the 16 MMA rows are (token, query head) pairs, 16 / G tokens per CTA,
// grid.x counts row tiles and every row carries its own causal bound.
// U8: the int8 tier (code - 128) * scale with one scale per cached row (napi/mod.rs:3474-3476): pages travel as bytes, a warp
// widens the page it is about to use to f16 integers in a staging page of its own, and the row scales multiply the score
// columns (K) and the probabilities before P V (V), so the tensor core only ever sees exact small integers.
template <int D, bool BF16, bool CHUNK, bool U8>
__global__ void __launch_bounds__(kAttnWarps * 32) attention_mma_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int PAGE_BYTES = kPageTokens * D * 2;               // one page as MMA operands (f16 / bf16)
  constexpr int RAW_PAGE = U8 ? kPageTokens * D : PAGE_BYTES;   // one page as cached
  constexpr int SCALE_BYTES = U8 ? kPageTokens * 4 : 0;         // its row scales
  constexpr int STAGE_BYTES = 2 * (RAW_PAGE + SCALE_BYTES);
  constexpr int WARP_BYTES = kAttnStages * STAGE_BYTES + (U8 ? 2 * PAGE_BYTES : 0);  // ring (+ the widened K and V page)
  constexpr int CHUNKS = D / 8;    // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;   // k16 steps of the QK^T product
  constexpr int DTILES = D / 8;    // n-tiles of the PV product
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  chain_wait();
  const int split = CHUNK ? 0 : blockIdx.x, kv_head = blockIdx.y, lane_id = blockIdx.z;
  const LaneInfo info = a.lanes[lane_id];
  const int G = a.q_heads / a.kv_heads;
  const int nsplits = CHUNK ? 1 : gridDim.x;
  // rows g and g + 8 of the MMA tile: which query token and head they are, and the positions [begin, end) they attend
  const int T = CHUNK ? a.tokens : 1;
  const int tokens_per_tile = CHUNK ? max(1, 16 / G) : 1;
  const int tile_token0 = CHUNK ? blockIdx.x * tokens_per_tile : 0;
  auto row_token = [&](int row) { return CHUNK ? tile_token0 + row / G : 0; };
  auto row_head = [&](int row) { return CHUNK ? row % G : row; };
  auto row_valid = [&](int row) { return CHUNK ? (row / G < tokens_per_tile && row_token(row) < T) : row < G; };
  auto row_end = [&](int row) { return CHUNK ? (row_valid(row) && info.advance > 0 ? info.cursor + row_token(row) + 1 : 0) : info.cursor + info.advance; };
  auto row_begin = [&](int row, int row_end_) {
    int b = info.start;
    if (a.op_window >= 0) b = max((int)max((long long)row_end_ - a.op_window, 0ll), info.start);
    return b;
  };
  const int end_lo = row_end(g), end_hi = row_end(g + 8);
  const int begin_lo = row_begin(g, end_lo), begin_hi = row_begin(g + 8, end_hi);
  // the tile as a whole: pages from the earliest begin to the latest end of its rows
  const int last_token = CHUNK ? min(T, tile_token0 + tokens_per_tile) - 1 : 0;
  const int end = CHUNK ? (info.advance > 0 && last_token >= tile_token0 ? info.cursor + last_token + 1 : 0) : info.cursor + info.advance;
  int begin = info.start;
  if (a.op_window >= 0) begin = max((int)max((long long)(CHUNK ? info.cursor + tile_token0 + 1 : end) - a.op_window, 0ll), info.start);
  const bool idle_lane = info.advance == 0 || end <= begin;
  // page range of this split (pages are indexed from the table start, i.e. position 0)
  const int first_page = begin / kPageTokens;
  const int last_page = idle_lane ? first_page : (end - 1) / kPageTokens + 1;  // exclusive
  const int p0 = first_page + split * a.pages_per_split;
  const int p1 = CHUNK ? last_page : min(last_page, p0 + a.pages_per_split);

  unsigned char* my_smem = smem + (size_t)warp * WARP_BYTES;
  unsigned char* wide = my_smem + kAttnStages * STAGE_BYTES;  // U8: this warp's widened K page, then V page
  const int* table = a.tables + info.table_offset;
  const size_t page_stride = (size_t)a.kv_heads * RAW_PAGE;  // bytes between consecutive pages
  const unsigned char* kbase = reinterpret_cast<const unsigned char*>(a.k) + (size_t)kv_head * RAW_PAGE;
  const unsigned char* vbase = reinterpret_cast<const unsigned char*>(a.v) + (size_t)kv_head * RAW_PAGE;

  auto issue = [&](int page_index, int stage) {
    if (page_index < p1) {
      const size_t off = (size_t)table[page_index] * page_stride;
      unsigned char* ks = my_smem + stage * STAGE_BYTES;
      unsigned char* vs = ks + RAW_PAGE;
      if (U8) {
        // bytes as they are (row-major), then the 16 row scales of K and of V
#pragma unroll
        for (int i = 0; i < RAW_PAGE / 16 / 32; ++i) {
          const int c = lane + 32 * i;
          cp_async16(ks + c * 16, kbase + off + (size_t)c * 16);
          cp_async16(vs + c * 16, vbase + off + (size_t)c * 16);
        }
        if (lane < 8) {
          const size_t si = ((size_t)table[page_index] * a.kv_heads + kv_head) * kPageTokens;  // 16 floats = 4 chunks each
          const float* src = (lane < 4 ? a.k_scale : a.v_scale) + si + (lane & 3) * 4;
          cp_async16(my_smem + stage * STAGE_BYTES + 2 * RAW_PAGE + lane * 16, src);
        }
      } else {
#pragma unroll
        for (int i = 0; i < (kPageTokens * CHUNKS) / 32; ++i) {
          const int c = lane + 32 * i;  // chunk index within the page
          const int row = c / CHUNKS, chunk = c % CHUNKS;
          const int so = swizzled_offset<D>(row, chunk);
          cp_async16(ks + so, kbase + off + (size_t)c * 16);
          cp_async16(vs + so, vbase + off + (size_t)c * 16);
        }
      }
    }
    cp_async_commit();  // always commit so group counting stays uniform
  };
  // U8: bytes of one cached page -> f16 integers (code - 128) in the swizzled operand layout
  auto widen = [&](const unsigned char* raw, unsigned char* dst) {
#pragma unroll
    for (int i = 0; i < RAW_PAGE / 16 / 32; ++i) {
      const int c = lane + 32 * i;  // 16 codes: row c / (D/16), columns 16 * (c % (D/16)) ...
      const int row = c / (D / 16), chunk = 2 * (c % (D / 16));
      const uint4 codes = *reinterpret_cast<const uint4*>(raw + c * 16);
      const uint32_t w[4] = {codes.x, codes.y, codes.z, codes.w};
      uint32_t h[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // bytes b0..b3 -> halves 1024 + b, minus 1152 = b - 128 (exact)
        const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
        uint32_t lo_bits = __byte_perm(w[j], 0x64646464u, 0x4140), hi_bits = __byte_perm(w[j], 0x64646464u, 0x4342);
        const __half2 lo = __hsub2(*reinterpret_cast<__half2*>(&lo_bits), bias);
        const __half2 hi = __hsub2(*reinterpret_cast<__half2*>(&hi_bits), bias);
        h[2 * j] = *reinterpret_cast<const uint32_t*>(&lo);
        h[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
      *reinterpret_cast<uint4*>(dst + swizzled_offset<D>(row, chunk)) = make_uint4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<uint4*>(dst + swizzled_offset<D>(row, chunk + 1)) = make_uint4(h[4], h[5], h[6], h[7]);
    }
  };

  // this warp's pages: p0 + warp, p0 + warp + 4, ...; the first copies are in flight while the query rows are fetched
  int next_issue = p0 + warp;
#pragma unroll
  for (int s = 0; s < kAttnStages - 1; ++s) {
    issue(next_issue, s);
    next_issue += kAttnWarps;
  }

  // Q fragments: rows 0..G-1 = query heads of this KV head, scaled into the exp2 domain
  uint32_t qf[KSTEPS][4];
  {
    const bool lo_ok = row_valid(g), hi_ok = row_valid(g + 8);
    const float* qrow_lo = a.q + (((size_t)lane_id * T + (lo_ok ? row_token(g) : 0)) * a.q_heads + kv_head * G + (lo_ok ? row_head(g) : 0)) * D;
    const float* qrow_hi = a.q + (((size_t)lane_id * T + (hi_ok ? row_token(g + 8) : 0)) * a.q_heads + kv_head * G + (hi_ok ? row_head(g + 8) : 0)) * D;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int c0 = ks * 16 + 2 * t;
      float2 x0 = lo_ok ? *reinterpret_cast<const float2*>(qrow_lo + c0) : make_float2(0.f, 0.f);
      float2 x1 = hi_ok ? *reinterpret_cast<const float2*>(qrow_hi + c0) : make_float2(0.f, 0.f);
      float2 x2 = lo_ok ? *reinterpret_cast<const float2*>(qrow_lo + c0 + 8) : make_float2(0.f, 0.f);
      float2 x3 = hi_ok ? *reinterpret_cast<const float2*>(qrow_hi + c0 + 8) : make_float2(0.f, 0.f);
      qf[ks][0] = pack2<BF16>(x0.x * a.scale_log2, x0.y * a.scale_log2);
      qf[ks][1] = pack2<BF16>(x1.x * a.scale_log2, x1.y * a.scale_log2);
      qf[ks][2] = pack2<BF16>(x2.x * a.scale_log2, x2.y * a.scale_log2);
      qf[ks][3] = pack2<BF16>(x3.x * a.scale_log2, x3.y * a.scale_log2);
    }
  }

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;  // rows g and g+8

  int stage = 0;
  for (int page_index = p0 + warp; page_index < p1; page_index += kAttnWarps) {
    issue(next_issue, (stage + kAttnStages - 1) % kAttnStages);
    next_issue += kAttnWarps;
    cp_async_wait<kAttnStages - 1>();
    __syncwarp();
    const unsigned char* ks_page = my_smem + stage * STAGE_BYTES;
    const unsigned char* vs_page = ks_page + RAW_PAGE;
    const float* page_scales = reinterpret_cast<const float*>(my_smem + stage * STAGE_BYTES + 2 * RAW_PAGE);  // U8: K rows, then V rows
    if (U8) {
      widen(ks_page, wide);
      widen(vs_page, wide + PAGE_BYTES);
      __syncwarp();
      ks_page = wide;
      vs_page = wide + PAGE_BYTES;
    }

    // S = Q K^T : two n-tiles of 8 tokens
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t kf[4];
      const int row = (lane & 7) + ((lane >> 4) << 3);
      const int chunk = 2 * ks + ((lane >> 3) & 1);
      ldmatrix_x4(kf, ks_page + swizzled_offset<D>(row, chunk));
      mma_16816<BF16>(s0, qf[ks], kf[0], kf[1]);
      mma_16816<BF16>(s1, qf[ks], kf[2], kf[3]);
    }
    if (U8) {  // score of token column c carries that cached row's K scale
      const float ka0 = page_scales[2 * t], ka1 = page_scales[2 * t + 1], kb0 = page_scales[2 * t + 8], kb1 = page_scales[2 * t + 9];
      s0[0] *= ka0; s0[1] *= ka1; s0[2] *= ka0; s0[3] *= ka1;
      s1[0] *= kb0; s1[1] *= kb1; s1[2] *= kb0; s1[3] *= kb1;
    }
    // mask positions outside [begin, end)
    const int base_pos = page_index * kPageTokens;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int pa = base_pos + 2 * t + j, pb = pa + 8;
      if (pa < begin_lo || pa >= end_lo) s0[j] = -INFINITY;
      if (pa < begin_hi || pa >= end_hi) s0[2 + j] = -INFINITY;
      if (pb < begin_lo || pb >= end_lo) s1[j] = -INFINITY;
      if (pb < begin_hi || pb >= end_hi) s1[2 + j] = -INFINITY;
    }
    // online softmax for rows g (index 0,1) and g+8 (index 2,3)
    float mx_lo = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
    float mx_hi = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    // a page with every position masked leaves the running maximum at -inf: keep factors finite
    const float alpha_lo = mn_lo == -INFINITY ? 1.0f : exp2f(m_lo - mn_lo);
    const float alpha_hi = mn_hi == -INFINITY ? 1.0f : exp2f(m_hi - mn_hi);
    const float sub_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, sub_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
    float p0v[4], p1v[4];
    p0v[0] = exp2f(s0[0] - sub_lo); p0v[1] = exp2f(s0[1] - sub_lo);
    p0v[2] = exp2f(s0[2] - sub_hi); p0v[3] = exp2f(s0[3] - sub_hi);
    p1v[0] = exp2f(s1[0] - sub_lo); p1v[1] = exp2f(s1[1] - sub_lo);
    p1v[2] = exp2f(s1[2] - sub_hi); p1v[3] = exp2f(s1[3] - sub_hi);
    l_lo = l_lo * alpha_lo + (p0v[0] + p0v[1] + p1v[0] + p1v[1]);
    l_hi = l_hi * alpha_hi + (p0v[2] + p0v[3] + p1v[2] + p1v[3]);
    m_lo = mn_lo; m_hi = mn_hi;
    if (U8) {  // V row scales ride on the probabilities; the denominators above stay unscaled
      const float* vsc = page_scales + kPageTokens;
      const float va0 = vsc[2 * t], va1 = vsc[2 * t + 1], vb0 = vsc[2 * t + 8], vb1 = vsc[2 * t + 9];
      p0v[0] *= va0; p0v[1] *= va1; p0v[2] *= va0; p0v[3] *= va1;
      p1v[0] *= vb0; p1v[1] *= vb1; p1v[2] *= vb0; p1v[3] *= vb1;
    }
    uint32_t pf[4];
    pf[0] = pack2<BF16>(p0v[0], p0v[1]);  // row g,   tokens 2t, 2t+1
    pf[1] = pack2<BF16>(p0v[2], p0v[3]);  // row g+8
    pf[2] = pack2<BF16>(p1v[0], p1v[1]);  // row g,   tokens 2t+8, 2t+9
    pf[3] = pack2<BF16>(p1v[2], p1v[3]);
    // O = O * alpha + P V
#pragma unroll
    for (int dp = 0; dp < DTILES / 2; ++dp) {
      uint32_t vf[4];
      const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = 2 * dp + (lane >> 4);
      ldmatrix_x4_trans(vf, vs_page + swizzled_offset<D>(row, chunk));
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float (&acc)[4] = o[2 * dp + j];
        acc[0] *= alpha_lo; acc[1] *= alpha_lo; acc[2] *= alpha_hi; acc[3] *= alpha_hi;
        mma_16816<BF16>(acc, pf, vf[2 * j], vf[2 * j + 1]);
      }
    }
    __syncwarp();
    stage = (stage + 1) % kAttnStages;
  }
  cp_async_wait<0>();
  // quad-reduce the denominators (each lane summed its own token columns)
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // ---- merge the 4 warps through shared memory (reusing the page ring)
  __syncthreads();
  float* mo = reinterpret_cast<float*>(smem);          // [warp][16 rows][D]
  float* mm = mo + kAttnWarps * 16 * D;                // [warp][16]
  float* ml = mm + kAttnWarps * 16;                    // [warp][16]
#pragma unroll
  for (int i = 0; i < DTILES; ++i) {
    float* lo = mo + ((size_t)warp * 16 + g) * D + i * 8 + 2 * t;
    float* hi = lo + 8 * D;
    lo[0] = o[i][0]; lo[1] = o[i][1];
    hi[0] = o[i][2]; hi[1] = o[i][3];
  }
  if (t == 0) {
    mm[warp * 16 + g] = m_lo; mm[warp * 16 + g + 8] = m_hi;
    ml[warp * 16 + g] = l_lo; ml[warp * 16 + g + 8] = l_hi;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < (CHUNK ? 16 : G) * D; idx += blockDim.x) {
    const int row = idx / D, d = idx - row * D;
    if (CHUNK && !row_valid(row)) continue;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) m = fmaxf(m, mm[w * 16 + row]);
    float acc = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float mw = mm[w * 16 + row];
      const float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
      acc += f * mo[((size_t)w * 16 + row) * D + d];
      l += f * ml[w * 16 + row];
    }
    const int head = kv_head * G + row_head(row);
    if (nsplits == 1) {
      const float val = l > 0.0f ? acc / l : 0.0f;
      a.out[(((size_t)lane_id * T + row_token(row)) * a.q_heads + head) * D + d] = val;
      if (!CHUNK && a.out_xh) {
        const int k = head * D + d;
        a.out_xh[((size_t)(k >> 3) * a.out_xh_nv + lane_id) * 8 + (k & 7)] = __float2half_rn(fminf(fmaxf(val, -65504.f), 65504.f));
      }
    } else {
      float* dst = a.partial + (((size_t)lane_id * a.q_heads + head) * nsplits + split) * (D + 2);
      dst[d] = acc;
      if (d == 0) { dst[D] = m; dst[D + 1] = l; }
    }
  }
}

// Combines split partials: out = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s. grid (Hq, B).
__global__ void attention_merge_kernel(const float* __restrict__ partial, int q_heads, int splits, int D,
                                       float* __restrict__ out, __half* __restrict__ out_xh, int xh_nv) {
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  chain_wait();
  const int head = blockIdx.x, lane_id = blockIdx.y;
  const float* base = partial + ((size_t)lane_id * q_heads + head) * splits * (D + 2);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, base[(size_t)s * (D + 2) + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.0f, l = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const float* p = base + (size_t)s * (D + 2);
      const float f = p[D] == -INFINITY ? 0.0f : exp2f(p[D] - m);
      acc += f * p[d];
      l += f * p[D + 1];
    }
    const float val = l > 0.0f ? acc / l : 0.0f;
    out[((size_t)lane_id * q_heads + head) * D + d] = val;
    if (out_xh) {
      const int k = head * D + d;
      out_xh[((size_t)(k >> 3) * xh_nv + lane_id) * 8 + (k & 7)] = __float2half_rn(fminf(fmaxf(val, -65504.f), 65504.f));
    }
  }
}

bool attention_mma_supported(const PoolView& pool, int q_heads, int tokens) {
  const int G = pool.kv_heads > 0 ? q_heads / pool.kv_heads : 0;
  return tokens >= 1 && pool.block_size == kPageTokens && (pool.head_dim == 64 || pool.head_dim == 128) &&
         (pool.dtype == kKvF16 || pool.dtype == kKvBF16 || pool.dtype == kKvU8) && G >= 1 && G <= 16 && q_heads % pool.kv_heads == 0;
}

AttnPlan plan_attention(int batch, int q_heads, int kv_heads, int head_dim, int max_pages, int sm_count) {
  AttnPlan p;
  const int ctas = std::max(1, batch * kv_heads);
  const int target = std::max(1, sm_count) * 2;
  int splits = std::max(1, target / ctas);
  // at least 2 pages per warp per split
  splits = std::min(splits, std::max(1, max_pages / (kAttnWarps * 2)));
  p.pages_per_split = std::max(1, (max_pages + splits - 1) / splits);
  p.splits = std::max(1, (max_pages + p.pages_per_split - 1) / p.pages_per_split);
  p.scratch_bytes = p.splits > 1 ? (size_t)batch * q_heads * p.splits * (head_dim + 2) * sizeof(float) : 0;
  return p;
}

size_t plan_attention_max_scratch(int batch, int q_heads, int kv_heads, int head_dim, int max_pages, int sm_count) {
  size_t need = 0;
  for (int pages = 1; pages <= max_pages; ++pages)
    need = std::max(need, plan_attention(batch, q_heads, kv_heads, head_dim, pages, sm_count).scratch_bytes);
  return need;
}

template <int D, bool BF16, bool CHUNK, bool U8>
static cudaError_t launch_attention_mma_t(const PoolView& pool, const AttnArgs& args, int batch, int grid_x,
                                          cudaStream_t stream) {
  constexpr size_t page = (size_t)kPageTokens * D * 2;
  constexpr size_t ring = U8 ? (size_t)kAttnWarps * (kAttnStages * 2 * (kPageTokens * D + kPageTokens * 4) + 2 * page)
                             : (size_t)kAttnWarps * kAttnStages * 2 * page;
  constexpr size_t merge = (size_t)kAttnWarps * 16 * (D + 2) * sizeof(float);
  constexpr size_t smem = ring > merge ? ring : merge;
  auto kernel = attention_mma_kernel<D, BF16, CHUNK, U8>;
  const cudaError_t attr = opt_in_shared_memory(kernel, smem);
  if (attr != cudaSuccess) return attr;
  dim3 grid((unsigned)grid_x, (unsigned)pool.kv_heads, (unsigned)batch);
  return launch_chained(kernel, grid, dim3(kAttnWarps * 32), smem, stream, args);
}

cudaError_t launch_attention_mma(const PoolView& pool, const float* q, const LaneInfo* lanes, const int* tables,
                                 int batch, int q_heads, double scale, long long op_window, float* out,
                                 const AttnPlan& plan, float* scratch, cudaStream_t stream, int* launches, __half* out_xh, int xh_nv,
                                 int tokens) {
  if (batch == 0) return cudaSuccess;
  if (batch > xh_nv || tokens > 1) out_xh = nullptr;
  AttnArgs args;
  args.out_xh = out_xh;
  args.out_xh_nv = xh_nv;
  args.k = pool.k; args.v = pool.v; args.q = q; args.lanes = lanes; args.tables = tables; args.out = out;
  args.partial = scratch; args.q_heads = q_heads; args.kv_heads = pool.kv_heads;
  args.pages_per_split = plan.pages_per_split;
  args.scale_log2 = (float)(scale * 1.4426950408889634);
  args.op_window = op_window;
  args.tokens = tokens;
  args.k_scale = pool.k_scale;
  args.v_scale = pool.v_scale;
  cudaError_t e;
  // the tier and the head width pick the instantiation; `chunk` the row mapping
  auto dispatch = [&](auto chunk_tag, int grid_x) {
    constexpr bool CHUNK = decltype(chunk_tag)::value;
    const bool wide = pool.head_dim == 128;
    if (pool.dtype == kKvU8)
      return wide ? launch_attention_mma_t<128, false, CHUNK, true>(pool, args, batch, grid_x, stream)
                  : launch_attention_mma_t<64, false, CHUNK, true>(pool, args, batch, grid_x, stream);
    if (pool.dtype == kKvBF16)
      return wide ? launch_attention_mma_t<128, true, CHUNK, false>(pool, args, batch, grid_x, stream)
                  : launch_attention_mma_t<64, true, CHUNK, false>(pool, args, batch, grid_x, stream);
    return wide ? launch_attention_mma_t<128, false, CHUNK, false>(pool, args, batch, grid_x, stream)
                : launch_attention_mma_t<64, false, CHUNK, false>(pool, args, batch, grid_x, stream);
  };
  if (tokens > 1) {
    // a prefill chunk: one CTA per tile of 16 / G tokens, no split over the pages
    const int G = q_heads / pool.kv_heads;
    const int per_tile = std::max(1, 16 / G);
    e = dispatch(std::true_type(), (tokens + per_tile - 1) / per_tile);
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
    return cudaSuccess;
  }
  e = dispatch(std::false_type(), plan.splits);
  if (e != cudaSuccess) return e;
  if (launches) ++*launches;
  if (plan.splits > 1) {
    dim3 grid((unsigned)q_heads, (unsigned)batch);
    e = launch_chained(attention_merge_kernel, grid, dim3((unsigned)std::min(128, pool.head_dim)), 0, stream, (const float*)scratch, q_heads, plan.splits,
                       pool.head_dim, out, out_xh, xh_nv);
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

// --------------------------------------------------------------------------------------------
// Fused RoPE + KV append. grid (q_heads + 2*kv_heads, batch, tokens), D/2 threads: token t of lane b is row b*tokens + t
// of qkv, sits at position cursor + t, and its rotated query goes to q_out[b, t, head, :].
// qkv row layout: [q heads | k heads | v heads] x D. Query heads are rotated into q_out, key heads
// are rotated and stored into the pool, value heads are stored. Angles in f64 like rope_kernel.
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ void pool_store(const PoolView& p, void* slab, size_t elem, float value) {
  if (p.dtype == kKvF32) reinterpret_cast<float*>(slab)[elem] = value;
  else if (p.dtype == kKvF16) reinterpret_cast<__half*>(slab)[elem] = __float2half_rn(value);
  else reinterpret_cast<__nv_bfloat16*>(slab)[elem] = __float2bfloat16_rn(value);
}

__global__ void rope_append_kernel(PoolView pool, const float* __restrict__ qkv, const LaneInfo* __restrict__ lanes,
                                   const int* __restrict__ tables, const double* __restrict__ inv_freq, int layout,
                                   int q_heads, float* __restrict__ q_out, DeferredSum sum) {
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  chain_wait();
  const int head = blockIdx.x, lane_id = blockIdx.y, tok = blockIdx.z, tokens = gridDim.z;
  const LaneInfo info = lanes[lane_id];
  const int D = pool.head_dim, half = D / 2;
  const int j = threadIdx.x;
  if (j >= half) return;
  const size_t row_width = (size_t)(q_heads + 2 * pool.kv_heads) * D;
  const size_t row = (size_t)lane_id * tokens + tok;
  const float* src = qkv + row * row_width + (size_t)head * D;
  const int i0 = layout == 0 ? j : 2 * j, i1 = layout == 0 ? half + j : 2 * j + 1;
  const bool is_q = head < q_heads, is_k = !is_q && head < q_heads + pool.kv_heads;
  float r0, r1;
  if (sum.splits > 0) {  // the projection left its split-K partials unsummed: add them up here, in split order
    // (a narrow shard of a tensor-parallel group has up to 32 splits: eight loads are in flight at a time)
    r0 = r1 = 0.f;
    const float* p = sum.partials + row * sum.rows_padded + (size_t)head * D;
    const size_t split_stride = (size_t)sum.vpad * sum.rows_padded;
    if (sum.splits <= 8) {
      for (int s = 0; s < sum.splits; ++s) {
        r0 += p[(size_t)s * split_stride + i0];
        r1 += p[(size_t)s * split_stride + i1];
      }
    } else for (int s0 = 0; s0 < sum.splits; s0 += 8) {
      float first[8], second[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool live = s0 + u < sum.splits;
        first[u] = live ? p[(size_t)(s0 + u) * split_stride + i0] : 0.f;
        second[u] = live ? p[(size_t)(s0 + u) * split_stride + i1] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (s0 + u < sum.splits) {
          r0 += first[u];
          r1 += second[u];
        }
      }
    }
  } else {
    r0 = src[i0];
    r1 = src[i1];
  }
  if (is_q || is_k) {
    const double angle = (double)(info.cursor + tok) * inv_freq[j];
    double s, c;
    sincos(angle, &s, &c);
    const double first = (double)r0, second = (double)r1;
    r0 = (float)__dsub_rn(__dmul_rn(first, c), __dmul_rn(second, s));
    r1 = (float)__dadd_rn(__dmul_rn(second, c), __dmul_rn(first, s));
  }
  if (is_q) {
    float* dst = q_out + (row * q_heads + head) * D;
    dst[i0] = r0;
    dst[i1] = r1;
    return;
  }
  if (info.advance == 0) return;  // padded lane: nothing is cached
  const int kv_head = is_k ? head - q_heads : head - q_heads - pool.kv_heads;
  const int pos = info.cursor + tok;
  const int page = tables[info.table_offset + pos / pool.block_size], slot = pos % pool.block_size;
  const size_t dst = pool_elem(pool, page, kv_head, slot);
  void* slab = is_k ? pool.k : pool.v;
  if (pool.dtype == kKvU8) {
    // the int8 tier: one scale per cached row, as kv_append_kernel (pool.rs:224-240)
    __shared__ float red[32];
    float amax = fmaxf(fabsf(r0), fabsf(r1));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) amax = fmaxf(amax, red[w]);
    const float scale = __fadd_rn(__fdiv_rn(amax, 127.0f), 1e-12f);
    if (threadIdx.x == 0) (is_k ? pool.k_scale : pool.v_scale)[pool_scale_index(pool, page, kv_head, slot)] = scale;
    const float c0 = fminf(fmaxf(roundf(__fdiv_rn(r0, scale)), -127.0f), 127.0f) + 128.0f;
    const float c1 = fminf(fmaxf(roundf(__fdiv_rn(r1, scale)), -127.0f), 127.0f) + 128.0f;
    reinterpret_cast<uint8_t*>(slab)[dst + i0] = (uint8_t)c0;
    reinterpret_cast<uint8_t*>(slab)[dst + i1] = (uint8_t)c1;
    return;
  }
  pool_store(pool, slab, dst + i0, r0);
  pool_store(pool, slab, dst + i1, r1);
}

cudaError_t launch_rope_append(const PoolView& pool, const float* qkv, const LaneInfo* lanes, const int* tables,
                               const double* inv_freq, int layout, int batch, int q_heads, float* q_out,
                               cudaStream_t stream, const DeferredSum* sum, int tokens) {
  if (batch == 0) return cudaSuccess;
  dim3 grid((unsigned)(q_heads + 2 * pool.kv_heads), (unsigned)batch, (unsigned)tokens);
  return launch_chained(rope_append_kernel, grid, dim3((unsigned)std::max(32, pool.head_dim / 2)), 0, stream, pool, qkv, lanes, tables, inv_freq, layout, q_heads,
                        q_out, sum ? *sum : DeferredSum());
}

__global__ void record_step_kernel(const uint32_t* __restrict__ tokens, uint32_t* __restrict__ ids,
                                   uint32_t* __restrict__ history, int* step_counter, LaneInfo* lanes, int64_t* cursors,
                                   int batch, long long window) {
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  chain_wait();
  const int step = *step_counter;
  for (int i = threadIdx.x; i < batch; i += blockDim.x) {
    const uint32_t tok = tokens[i];
    ids[i] = tok;
    history[(size_t)step * batch + i] = tok;
    if (lanes[i].advance > 0) {
      lanes[i].cursor += 1;
      cursors[i] += 1;
      if (window >= 0) lanes[i].start = (int)max((long long)lanes[i].cursor + 1 - window, 0ll);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *step_counter = step + 1;
}
cudaError_t launch_record_step(const uint32_t* tokens, uint32_t* ids, uint32_t* history, int* step_counter, LaneInfo* lanes,
                               int64_t* cursors, int batch, long long window, cudaStream_t stream) {
  return launch_chained(record_step_kernel, dim3(1), dim3(128), 0, stream, tokens, ids, history, step_counter, lanes, cursors, batch, window);
}

// Debug/test read-back of logical token rows (row = block*block_size + offset) as f32
// [n, kv_heads*head_dim] in the reference's row order, dequantised for the u8 tier.
__global__ void pool_read_rows_kernel(PoolView pool, const uint32_t* __restrict__ rows, int64_t n, float* __restrict__ out,
                                      int which) {
  const int64_t width = (int64_t)pool.kv_heads * pool.head_dim;
  const int64_t total = n * width;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = idx / width, e = idx - i * width;
    const int head = (int)(e / pool.head_dim), d = (int)(e % pool.head_dim);
    const int page = (int)(rows[i] / pool.block_size), slot = (int)(rows[i] % pool.block_size);
    out[idx] = pool_load(pool, which == 0 ? pool.k : pool.v, which == 0 ? pool.k_scale : pool.v_scale,
                         pool_elem(pool, page, head, slot) + d, pool_scale_index(pool, page, head, slot));
  }
}
cudaError_t launch_pool_read_rows(const PoolView& pool, const uint32_t* rows, int64_t n, float* out, int which,
                                  cudaStream_t stream) {
  const int64_t total = n * pool.kv_heads * pool.head_dim;
  if (total == 0) return cudaSuccess;
  pool_read_rows_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8), 256, 0, stream>>>(pool, rows, n, out, which);
  return cudaGetLastError();
}

}  // namespace etc
