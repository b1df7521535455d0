// Decode-shaped dequant linear on tcgen05 for Q4_0 / Q8_0 weights: few input vectors (<= 128), weights streamed once.
//
//   out[v, r] = sum_k x[v, k] * deq(W[r, k])        (quantized_linear, crates/runtime-cpu/src/quantized.rs:419-499)
//
// One tcgen05.mma costs about a hundred cycles however small it is, and its duration grows only with N. So the
// WEIGHTS take the N side at its maximum (256 rows per instruction) and the input vectors the M side:
//   * B operand = 256 weight rows x 16 columns, f16 in shared memory (canonical K-major, no swizzle). Eight dequant
//     warps own one weight row per thread: they read the row's packed block from a ring that bulk copies fill
//     straight from HBM, expand it to f16 in registers (times the block scale) and store 16-byte groups, which
//     land conflict-free because consecutive rows are consecutive 16-byte slots of a core matrix.
//   * A operand = the input vectors, one per TENSOR MEMORY lane, two f16 columns per 32-bit TMEM column; a loader
//     warp per 32 vectors moves them from the bulk-copied stage (the producer's f16 layout, [K/8][vectors][8]) with tcgen05.st.
//   * D = f32 [vectors x 256 rows] in tensor memory: lane = vector, column = weight row.
// Work is cut stream-K style: the (tile, 64-column stage) units of the whole matrix are numbered tile-major and
// every CTA (one per SM) takes one contiguous range, so all SMs stream the same number of bytes whatever the
// matrix shape. A range that covers a whole tile finishes it in place (bias, residual add, SwiGLU over
// interleaved gate/up rows, optional f16 copy for the next linear); a partial range stores f32 partial sums and
// the last CTA to arrive at the tile (one atomic ticket, no waiting) adds all of them in a fixed order.
//
// Warp roles: 16 dequant warps, activation loaders (one per 32 vectors), epilogue warps (one per 32 vectors), one
// bulk-copy issuing lane, one MMA issuing lane. Rings: bulk-copied packed weights + activations (smem, 2-7
// stages), f16 weights (smem, 4), activations (TMEM, 4); tcgen05.commit frees a stage when the MMAs that read it have retired.
//
// Every mbarrier wait is bounded: on expiry the thread raises the abort flag and the status word, all roles fall
// through to the teardown, tensor memory is freed and the kernel returns.
//
// Roofline: HBM-bound by bytes = rows*K/32*{18,34} + 2*vectors*K + 4*vectors*rows; the tensor pipe allows about
// 30 weights per cycle per SM at this shape, some 70% of what HBM could deliver for Q4_0.
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.h"
#include "tc05.cuh"

namespace etc {

namespace {

using namespace tc05;

constexpr int kTileRows = 256;       // weight rows per tile = MMA N
constexpr int kStageBlocks = 2;      // 32-value blocks per stage; one stage = one unit of stream-K work
constexpr int kStages = 4;           // operand stages: f16 weights in shared memory + activations in tensor memory (32 columns)
constexpr int kDequantWarps = 16;  // two groups of 8 warps take alternate stages, one weight row per thread; arrivals are per warp
constexpr int kGroupWarps = 8;
constexpr int kOwnSumMaxRanges = 3;   // tiles cut into more ranges than this are summed by a second kernel
// Warp roles. A warp reaches the 32 TMEM lanes of its index modulo 4, so loader and epilogue warps sit at multiples
// of 4 plus the vector group they serve. With one vector group (LW = 1) the CTA is 21 warps, else 26.
template <int LW>
struct StreamRoles {
  static constexpr int kLoaderWarp0 = 16;
  static constexpr int kEpilogueWarp0 = 20;
  static constexpr int kCopyWarp = LW == 1 ? 17 : 24;
  static constexpr int kMmaWarp = LW == 1 ? 18 : 25;
  static constexpr int kWarps = LW == 1 ? 21 : 26;
  static constexpr int kThreads = kWarps * 32;
};
constexpr uint32_t kKGroupBytes = kTileRows * 16;                 // 8 columns of all 256 rows (descriptor LBO)
constexpr uint32_t kBlockHalfBytes = 4 * kKGroupBytes;            // one 32-value block as f16
constexpr uint32_t kStageBBytes = kStageBlocks * kBlockHalfBytes;
constexpr uint32_t kTmemCols = 512;                               // D: columns [0, 256); activations: [256, 512)
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kTileRows >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);  // f16 x f16 -> f32

template <int CODEC, int LW>
struct StreamCfg {
  static constexpr int kQuantBytes = CODEC == 2 ? 16 : 32;                       // packed payload per row and block
  static constexpr uint32_t kChunkBytes = kTileRows * (kQuantBytes + 2);         // 256 rows' payload, then their scales
  static constexpr uint32_t kStageWBytes = kStageBlocks * kChunkBytes;
  static constexpr uint32_t kStageXBytes = LW * 32 * kStageBlocks * 32 * 2;      // the stage's activations, [8 column groups][vectors][8] f16
  static constexpr uint32_t kRingStageBytes = kStageWBytes + kStageXBytes;       // one bulk-copied stage: packed weights, then activations
  static constexpr int kWStages = LW == 1 ? (CODEC == 2 ? 7 : 4) : (CODEC == 2 ? 3 : 2);
  static constexpr int kBarriers = 2 * kWStages + 2 * kStages + 2;
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBBytes + (size_t)kWStages * kRingStageBytes + kBarriers * sizeof(uint64_t) + 16;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

struct StreamArgs {
  const unsigned char* weights;  // [tile][kblock] chunks
  const __half* xh;              // [K/8][nvp][8] f16
  const float* bias;
  const float* residual;
  float* out;
  __half* out_xh;                // optional f16 copy of the result, [out_cols/8][out_xh_nv][8]
  float* partials;               // [slots][nvp][256] f32
  int* counters;                 // [tiles][4], zero between launches
  unsigned long long* status;
  int out_xh_nv;
  int vectors, nvp, rows, tiles, spt, total_units, units_per_cta, epilogue, slot_mode;
  int own_sum;  // 1: the last CTA to reach a tile adds up its partial sums; 0: qlinear_stream_sum_kernel does, afterwards
};

// Partial-sum slot of CTA c's range inside tile t. Mode 0: two slots per CTA (the range's first tile, any later one);
// mode 1: c + t, unique because both only grow along the unit order. The host picks the smaller table.
__device__ __forceinline__ int partial_slot(const StreamArgs& a, int c, int t) {
  if (a.slot_mode == 1) return c + t;
  return 2 * c + (t != (c * a.units_per_cta) / a.spt ? 1 : 0);
}

__device__ __forceinline__ uint32_t pack_half2_sat(float x, float y) {
  return h2u(__floats2half2_rn(fminf(fmaxf(x, -65504.f), 65504.f), fminf(fmaxf(y, -65504.f), 65504.f)));
}

// Finishes 16 consecutive (padded) rows rb..rb+15 of vector v; rb is a multiple of 16.
__device__ __forceinline__ void emit_rows16(const StreamArgs& a, const float (&val)[16], int rb, int v) {
  if (v >= a.vectors) return;
  if (a.epilogue == ETC_EPILOGUE_SWIGLU) {
    // rows are interleaved in groups of 8: rows 0-7 of the 16 are gate rows and rows 8-15 their up rows
    const int out_cols = a.rows >> 1, oc0 = (rb >> 4) * 8;
    float act[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool live = rb + j + 8 < a.rows;
      const float g = val[j] + (a.bias && live ? a.bias[rb + j] : 0.0f);
      const float u = val[8 + j] + (a.bias && live ? a.bias[rb + j + 8] : 0.0f);
      act[j] = silu_tanh(g) * u;
    }
    if (rb + 16 <= a.rows && (out_cols & 7) == 0) {
      if (a.out) {
        float4* dst = reinterpret_cast<float4*>(a.out + (size_t)v * out_cols + oc0);
        dst[0] = make_float4(act[0], act[1], act[2], act[3]);
        dst[1] = make_float4(act[4], act[5], act[6], act[7]);
      }
      if (a.out_xh)
        reinterpret_cast<uint4*>(a.out_xh)[(size_t)(oc0 >> 3) * a.out_xh_nv + v] =
            make_uint4(pack_half2_sat(act[0], act[1]), pack_half2_sat(act[2], act[3]), pack_half2_sat(act[4], act[5]), pack_half2_sat(act[6], act[7]));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (rb + j + 8 >= a.rows) continue;
        const int oc = oc0 + j;
        if (a.out) a.out[(size_t)v * out_cols + oc] = act[j];
        if (a.out_xh) a.out_xh[((size_t)(oc >> 3) * a.out_xh_nv + v) * 8 + (oc & 7)] = __float2half_rn(fminf(fmaxf(act[j], -65504.f), 65504.f));
      }
    }
    return;
  }
  const bool add = a.epilogue == ETC_EPILOGUE_RESIDUAL;
  if (rb + 16 <= a.rows && (a.rows & 7) == 0) {
    float* dst = a.out + (size_t)v * a.rows + rb;
    const float* res = add ? a.residual + (size_t)v * a.rows + rb : nullptr;
    float x[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (add) r4 = *reinterpret_cast<const float4*>(res + 4 * q);
      const float r[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float y = val[4 * q + e] + (a.bias ? a.bias[rb + 4 * q + e] : 0.0f);  // scalar: a caller's bias need not be 16-byte aligned
        if (add) y = r[e] + y;
        x[4 * q + e] = y;
      }
      reinterpret_cast<float4*>(dst)[q] = make_float4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
    }
    if (a.out_xh) {
#pragma unroll
      for (int g = 0; g < 2; ++g)
        reinterpret_cast<uint4*>(a.out_xh)[(size_t)((rb >> 3) + g) * a.out_xh_nv + v] =
            make_uint4(pack_half2_sat(x[8 * g], x[8 * g + 1]), pack_half2_sat(x[8 * g + 2], x[8 * g + 3]),
                       pack_half2_sat(x[8 * g + 4], x[8 * g + 5]), pack_half2_sat(x[8 * g + 6], x[8 * g + 7]));
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int r = rb + j;
    if (r >= a.rows) continue;
    const size_t o = (size_t)v * a.rows + r;
    float x = val[j] + (a.bias ? a.bias[r] : 0.0f);
    if (add) x = a.residual[o] + x;
    a.out[o] = x;
    if (a.out_xh) a.out_xh[((size_t)(r >> 3) * a.out_xh_nv + v) * 8 + (r & 7)] = __float2half_rn(fminf(fmaxf(x, -65504.f), 65504.f));
  }
}

// Adds up the partial sums of 16 rows (group g of the tile) for vector v over the CTAs c_first..c_last, in CTA order,
// and finishes the rows. MAXSEG > 0: at most that many ranges, all loads in flight at once.
template <int MAXSEG>
__device__ __forceinline__ void sum_partials16(const StreamArgs& a, int tile, int c_first, int c_last, int v, int g) {
  float val[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) val[j] = 0.0f;
  if (MAXSEG > 0) {
    float4 p[MAXSEG > 0 ? MAXSEG : 1][4];
#pragma unroll
    for (int s = 0; s < MAXSEG; ++s) {
      const int c = min(c_first + s, c_last);
      const float4* theirs = reinterpret_cast<const float4*>(a.partials + ((size_t)partial_slot(a, c, tile) * a.nvp + v) * kTileRows + g * 16);
#pragma unroll
      for (int q = 0; q < 4; ++q) p[s][q] = __ldcg(theirs + q);
    }
#pragma unroll
    for (int s = 0; s < MAXSEG; ++s) {
      if (c_first + s > c_last) break;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        val[4 * q] += p[s][q].x; val[4 * q + 1] += p[s][q].y; val[4 * q + 2] += p[s][q].z; val[4 * q + 3] += p[s][q].w;
      }
    }
  } else {
#pragma unroll 4
    for (int c = c_first; c <= c_last; ++c) {
      const float4* theirs = reinterpret_cast<const float4*>(a.partials + ((size_t)partial_slot(a, c, tile) * a.nvp + v) * kTileRows + g * 16);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 p = __ldcg(theirs + q);
        val[4 * q] += p.x; val[4 * q + 1] += p.y; val[4 * q + 2] += p.z; val[4 * q + 3] += p.w;
      }
    }
  }
  emit_rows16(a, val, tile * kTileRows + g * 16, v);
}

// Second pass for matrices whose tiles are cut into many ranges: one CTA per (tile, 32 vectors), 512 threads.
__global__ void __launch_bounds__(512) qlinear_stream_sum_kernel(StreamArgs a) {
  const int tile = blockIdx.x, lw = blockIdx.y;
  const int c_first = (tile * a.spt) / a.units_per_cta;
  const int c_last = ((tile + 1) * a.spt - 1) / a.units_per_cta;
  if (c_first == c_last) return;  // a single CTA covered the tile and finished it in place
  sum_partials16<0>(a, tile, c_first, c_last, lw * 32 + (threadIdx.x >> 4), threadIdx.x & 15);
}

template <int CODEC, int LW>
__global__ void __launch_bounds__(StreamRoles<LW>::kThreads, 1) qlinear_stream_kernel(StreamArgs a) {
  using Cfg = StreamCfg<CODEC, LW>;
  using Roles = StreamRoles<LW>;
  constexpr int kLoaderWarp0 = Roles::kLoaderWarp0, kEpilogueWarp0 = Roles::kEpilogueWarp0;
  constexpr int kCopyWarp = Roles::kCopyWarp, kMmaWarp = Roles::kMmaWarp;
  constexpr int kWStages = Cfg::kWStages;
  constexpr int QW = CODEC == 2 ? 1 : 2;  // uint4 words per (row, block)
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* b_ring = smem;                                   // kStages * kStageBBytes, f16 weights
  unsigned char* w_ring = smem + kStages * kStageBBytes;          // kWStages * kRingStageBytes, bulk-copied packed weights + activations
  uint64_t* full_w = reinterpret_cast<uint64_t*>(w_ring + (size_t)kWStages * Cfg::kRingStageBytes);
  uint64_t* empty_w = full_w + kWStages;   // one arrival per warp of the group: packed stage consumed into registers
  uint64_t* full = empty_w + kWStages;     // one arrival per warp of the group and per loader warp: both operands stored
  uint64_t* empty = full + kStages;        // tcgen05.commit: the MMAs that read the stage have retired
  uint64_t* d_full = empty + kStages;      // tcgen05.commit: accumulator of a range complete
  uint64_t* d_empty = d_full + 1;          // one arrival per epilogue warp: accumulator read out
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(d_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  __shared__ int pending_tile[4][2];  // tiles whose partial sums this CTA must add up at the end, per 32-vector group
  __shared__ int pending_count[4];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lanewarps = a.nvp >> 5;
  const int u0 = blockIdx.x * a.units_per_cta;
  const int n = min(a.total_units, u0 + a.units_per_cta) - u0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWStages; ++s) {
      mbar_init(&full_w[s], 1);
      mbar_init(&empty_w[s], kGroupWarps + lanewarps);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], kGroupWarps + lanewarps);
      mbar_init(&empty[s], 1);
    }
    mbar_init(d_full, 1);
    mbar_init(d_empty, lanewarps);
    for (int e = 0; e < 4; ++e) pending_count[e] = 0;
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(tmem_holder, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t d_tmem = tmem_base;           // columns [0, 256)
  const uint32_t a_tmem0 = tmem_base + 256;    // stage s at columns 256 + 32 s

  if (warp < kDequantWarps) {
    // ------------------------------------------------------------------ dequant warps: one weight row per thread,
    // the two groups take alternate stages so that one group's waits hide behind the other group's work
    const int row = threadIdx.x & (kTileRows - 1);
    for (int i = warp / kGroupWarps; i < n; i += kDequantWarps / kGroupWarps) {
      const int sw = i % kWStages, st = i % kStages;
      if (!mbar_wait_warp(&full_w[sw], (uint32_t)(i / kWStages) & 1, abort_flag)) break;
      const unsigned char* ws = w_ring + (size_t)sw * Cfg::kRingStageBytes;
      uint4 q[kStageBlocks][QW];
      __half sc[kStageBlocks];
#pragma unroll
      for (int b = 0; b < kStageBlocks; ++b) {
        const unsigned char* chunk = ws + (size_t)b * Cfg::kChunkBytes;
#pragma unroll
        for (int w = 0; w < QW; ++w) q[b][w] = *reinterpret_cast<const uint4*>(chunk + ((size_t)w * kTileRows + row) * 16);
        sc[b] = *reinterpret_cast<const __half*>(chunk + kTileRows * Cfg::kQuantBytes + row * 2);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_w[sw]);  // the warp's part of the packed stage now lives in registers
      uint32_t regs[kStageBlocks][16];
#pragma unroll
      for (int b = 0; b < kStageBlocks; ++b) {
        const __half2 s2 = __half2half2(sc[b]);
        if (CODEC == 2) {
          expand_q4(q[b][0].x, s2, regs[b] + 0);
          expand_q4(q[b][0].y, s2, regs[b] + 4);
          expand_q4(q[b][0].z, s2, regs[b] + 8);
          expand_q4(q[b][0].w, s2, regs[b] + 12);
        } else {
          const uint4 q0 = q[b][0], q1 = q[b][QW - 1];
          expand_q8(q0.x, s2, regs[b] + 0); expand_q8(q0.y, s2, regs[b] + 2); expand_q8(q0.z, s2, regs[b] + 4); expand_q8(q0.w, s2, regs[b] + 6);
          expand_q8(q1.x, s2, regs[b] + 8); expand_q8(q1.y, s2, regs[b] + 10); expand_q8(q1.z, s2, regs[b] + 12); expand_q8(q1.w, s2, regs[b] + 14);
        }
      }
      // the MMAs that read this stage in the previous round must have retired
      if (!mbar_wait_warp(&empty[st], ((uint32_t)(i / kStages) & 1) ^ 1, abort_flag)) break;
      unsigned char* dst = b_ring + (size_t)st * kStageBBytes + (size_t)row * 16;
#pragma unroll
      for (int b = 0; b < kStageBlocks; ++b)
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(dst + (size_t)b * kBlockHalfBytes + (size_t)g * kKGroupBytes) =
              make_uint4(regs[b][4 * g], regs[b][4 * g + 1], regs[b][4 * g + 2], regs[b][4 * g + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[st]);
    }
  } else if (warp >= kLoaderWarp0 && warp < kLoaderWarp0 + LW) {
    // ------------------------------------------------------------------ activation loaders: one vector per thread
    const int lw = warp - kLoaderWarp0;
    if (lw < lanewarps && lw < LW) {
      const int v = lw * 32 + lane;
      const uint32_t lane_base = (uint32_t)(lw * 32) << 16;
      for (int i = 0; i < n; ++i) {
        const int sw = i % kWStages, st = i % kStages;
        if (!mbar_wait_warp(&full_w[sw], (uint32_t)(i / kWStages) & 1, abort_flag)) break;
        const uint4* src = reinterpret_cast<const uint4*>(w_ring + (size_t)sw * Cfg::kRingStageBytes + Cfg::kStageWBytes) + v;
        uint32_t x[2][16];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint4 x4 = src[(size_t)g * a.nvp];
          x[g >> 2][(g & 3) * 4 + 0] = x4.x; x[g >> 2][(g & 3) * 4 + 1] = x4.y;
          x[g >> 2][(g & 3) * 4 + 2] = x4.z; x[g >> 2][(g & 3) * 4 + 3] = x4.w;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_w[sw]);
        if (!mbar_wait_warp(&empty[st], ((uint32_t)(i / kStages) & 1) ^ 1, abort_flag)) break;
        tc_fence_after();
        tmem_st16(a_tmem0 + lane_base + (uint32_t)(st * 32), x[0]);
        tmem_st16(a_tmem0 + lane_base + (uint32_t)(st * 32 + 16), x[1]);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[st]);
      }
    }
  } else if (warp >= kEpilogueWarp0 && warp < kEpilogueWarp0 + LW) {
    // ------------------------------------------------------------------ epilogue: one vector per thread
    const int lw = warp - kEpilogueWarp0;
    if (lw < lanewarps) {
      const int v = lw * 32 + lane;
      const uint32_t lane_base = (uint32_t)(lw * 32) << 16;
      int seg = 0;
      for (int i = 0; i < n; ++seg) {
        const int u = u0 + i, tile = u / a.spt, ks0 = u - tile * a.spt;
        const int len = min(a.spt - ks0, n - i);
        i += len;
        if (!mbar_wait_warp(d_full, (uint32_t)seg & 1, abort_flag)) break;
        tc_fence_after();
        if (len == a.spt) {
#pragma unroll 1
          for (int c0 = 0; c0 < kTileRows; c0 += 16) {
            uint32_t acc[16];
            tmem_ld16(d_tmem + lane_base + (uint32_t)c0, acc);
            tmem_wait_ld();
            float val[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) val[j] = __uint_as_float(acc[j]);
            emit_rows16(a, val, tile * kTileRows + c0, v);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(d_empty);
          continue;
        }
        float* mine = a.partials + ((size_t)partial_slot(a, blockIdx.x, tile) * a.nvp + v) * kTileRows;
#pragma unroll 1
        for (int c0 = 0; c0 < kTileRows; c0 += 16) {
          uint32_t acc[16];
          tmem_ld16(d_tmem + lane_base + (uint32_t)c0, acc);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 4; ++q)
            reinterpret_cast<uint4*>(mine + c0)[q] = make_uint4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
        }
        tc_fence_before();
        __threadfence();
        __syncwarp();
        // one ticket per (tile, 32-vector group): whoever draws the last one adds up every range's partial sums,
        // with the whole CTA, after its own ranges are done
        if (lane == 0) {
          mbar_arrive(d_empty);  // the next range's MMAs may overwrite the accumulator now
          if (!a.own_sum) continue;
          const int c_first = (tile * a.spt) / a.units_per_cta;
          const int c_last = ((tile + 1) * a.spt - 1) / a.units_per_cta;
          if (atomicAdd(&a.counters[tile * 4 + lw], 1) == c_last - c_first) {
            __threadfence();
            pending_tile[lw][pending_count[lw]++] = tile;
          }
        }
      }
    }
  } else if (warp == kCopyWarp) {
    // ------------------------------------------------------------------ bulk copies: this CTA's units are one contiguous byte range
    if (lane == 0) {
      const unsigned char* src = a.weights + (size_t)u0 * Cfg::kStageWBytes;
      const uint32_t x_bytes = (uint32_t)a.nvp * (kStageBlocks * 32 * 2);  // this stage's activations: 8 column groups x nvp x 16 bytes
      int issued = 0;
      for (int i = 0; i < n; ++i) {
        const int sw = i % kWStages;
        if (!mbar_wait(&empty_w[sw], ((uint32_t)(i / kWStages) & 1) ^ 1, abort_flag)) break;
        unsigned char* dst = w_ring + (size_t)sw * Cfg::kRingStageBytes;
        const int ks = (u0 + i) % a.spt;
        mbar_arrive_expect_tx(&full_w[sw], Cfg::kStageWBytes + x_bytes);
        bulk_copy_g2s(dst, src + (size_t)i * Cfg::kStageWBytes, Cfg::kStageWBytes, &full_w[sw]);
        bulk_copy_g2s(dst + Cfg::kStageWBytes, reinterpret_cast<const unsigned char*>(a.xh) + (size_t)ks * x_bytes, x_bytes, &full_w[sw]);
        issued = i + 1;
      }
      if (*abort_flag) {
        // give-up path: let this thread's own bulk copies land (bounded) before shared memory is released
        for (int i = max(0, issued - kWStages); i < issued; ++i)
          for (unsigned spin = 0; spin < (1u << 20) && !mbar_try_wait(&full_w[i % kWStages], (uint32_t)(i / kWStages) & 1); ++spin) __nanosleep(64);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      int seg = 0;
      for (int i = 0; i < n; ++i) {
        const int ks = (u0 + i) % a.spt;
        const int st = i % kStages;
        const bool first = i == 0 || ks == 0;
        if (!mbar_wait(&full[st], (uint32_t)(i / kStages) & 1, abort_flag)) break;
        if (first && !mbar_wait(d_empty, ((uint32_t)seg & 1) ^ 1, abort_flag)) break;  // previous range read out
        tc_fence_after();
        const uint32_t b_base = smem_u32(b_ring + (size_t)st * kStageBBytes);
#pragma unroll
        for (int j = 0; j < 2 * kStageBlocks; ++j) {  // K = 16 per MMA: two 8-column groups of B, 8 TMEM columns of A
          const uint64_t b_desc = make_b_desc(b_base + (uint32_t)j * 2u * kKGroupBytes, kKGroupBytes, 128u);
          umma_ts(d_tmem, a_tmem0 + (uint32_t)(st * 32 + j * 8), b_desc, kIdesc, (first && j == 0) ? 0u : 1u);
        }
        tc_commit(&empty[st]);  // arrives when the MMAs above have finished reading their operands
        if (ks == a.spt - 1 || i == n - 1) {
          tc_commit(d_full);
          ++seg;
        }
      }
      tc_fence_before();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(a.status, 0ull, 3ull);  // bounded wait expired
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  // ------------------------------------------------------------------ tiles this CTA was the last to reach
  // 32 vectors x 16 groups of 16 rows = 512 work items per (tile, vector group); every range's partial sums are
  // added in CTA order, so the result does not depend on who arrived last.
  if (*abort_flag) return;
  for (int lw = 0; lw < lanewarps; ++lw) {
    for (int e = 0; e < pending_count[lw]; ++e) {
      const int tile = pending_tile[lw][e];
      const int c_first = (tile * a.spt) / a.units_per_cta;
      const int c_last = ((tile + 1) * a.spt - 1) / a.units_per_cta;
      if (threadIdx.x < 512)  // the dequant warps' threads; in this mode a tile has at most kOwnSumMaxRanges ranges
        sum_partials16<kOwnSumMaxRanges>(a, tile, c_first, c_last, lw * 32 + (threadIdx.x >> 4), threadIdx.x & 15);
      if (threadIdx.x == 0) a.counters[tile * 4 + lw] = 0;  // ready for the next launch
    }
  }
}

// f32 [vectors, K] -> f16 [K/8][nvp][8] (rows >= vectors are zero), saturating like the other tensor-core paths.
__global__ void convert_xh8_rows_kernel(const float* __restrict__ x, int vectors, int K, int nvp, __half* __restrict__ xh) {
  const int total = (K / 8) * nvp;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int kg = idx / nvp, v = idx - kg * nvp;
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (v < vectors) {
      const float4 lo = *reinterpret_cast<const float4*>(x + (size_t)v * K + kg * 8);
      const float4 hi = *reinterpret_cast<const float4*>(x + (size_t)v * K + kg * 8 + 4);
      auto sat = [](float y) { return fminf(fmaxf(y, -65504.f), 65504.f); };
      packed.x = h2u(__floats2half2_rn(sat(lo.x), sat(lo.y)));
      packed.y = h2u(__floats2half2_rn(sat(lo.z), sat(lo.w)));
      packed.z = h2u(__floats2half2_rn(sat(hi.x), sat(hi.y)));
      packed.w = h2u(__floats2half2_rn(sat(hi.z), sat(hi.w)));
    }
    reinterpret_cast<uint4*>(xh)[idx] = packed;
  }
}

// Raw GGUF rows -> [tile of 256 rows][block] chunks. A chunk holds the 256 rows' packed payload (16 bytes per row
// for Q4_0 with nibbles reordered for expand_q4; for Q8_0 two 16-byte halves, half-major) followed by their 256
// f16 scales, so that a stage of the kernel is one contiguous bulk copy. Rows beyond `rows` decode to zero.
__global__ void repack_stream_kernel(RepackParts parts, int codec, int64_t rows, int64_t rows_padded, int64_t kblocks,
                                     int interleave8, unsigned char* __restrict__ dst_base) {
  const int64_t total = rows_padded * kblocks;
  const int bb = codec == 2 ? 18 : 34;
  const int qb = codec == 2 ? 16 : 32;
  const int64_t chunk_bytes = (int64_t)kTileRows * (qb + 2);
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / kblocks, kb = idx - r * kblocks;
    const uint8_t* src_row = nullptr;
    if (r < rows) {
      if (interleave8) {
        const int64_t grp = r >> 4, within = r & 15;
        src_row = parts.ptr[within >= 8 ? 1 : 0] + (grp * 8 + (within & 7)) * kblocks * bb;
      } else {
        int64_t rr = r;
        for (int p = 0; p < parts.n_parts; ++p) {
          if (rr < parts.rows[p]) { src_row = parts.ptr[p] + rr * kblocks * bb; break; }
          rr -= parts.rows[p];
        }
      }
    }
    const int64_t tile = r / kTileRows, row = r % kTileRows;
    unsigned char* chunk = dst_base + (tile * kblocks + kb) * chunk_bytes;
    uint32_t words[8];
    __half scale = __float2half_rn(0.0f);
    if (!src_row) {
      for (int w = 0; w < 8; ++w) words[w] = codec == 2 ? 0x88888888u : 0u;
    } else {
      const uint8_t* blk = src_row + kb * bb;
      scale = __ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8)));
      if (codec == 2) {
        const int pos[8] = {0, 16, 8, 24, 4, 20, 12, 28};
        for (int w = 0; w < 4; ++w) {
          uint32_t word = 0;
          for (int j = 0; j < 8; ++j) {
            const int i = 8 * w + j;
            const uint32_t code = i < 16 ? (blk[2 + i] & 0x0fu) : (uint32_t)(blk[2 + i - 16] >> 4);
            word |= code << pos[j];
          }
          words[w] = word;
        }
      } else {
        for (int w = 0; w < 8; ++w) {
          uint32_t word = 0;
          for (int j = 0; j < 4; ++j) word |= (uint32_t)blk[2 + 4 * w + j] << (8 * j);
          words[w] = word;
        }
      }
    }
    const int halves = codec == 2 ? 1 : 2;
    for (int h = 0; h < halves; ++h)
      *reinterpret_cast<uint4*>(chunk + ((int64_t)h * kTileRows + row) * 16) = make_uint4(words[4 * h], words[4 * h + 1], words[4 * h + 2], words[4 * h + 3]);
    *reinterpret_cast<__half*>(chunk + (int64_t)kTileRows * qb + row * 2) = scale;
  }
}

template <int CODEC, int LW>
cudaError_t launch_stream_pass(const StreamArgs& args, int grid, cudaStream_t stream) {
  constexpr size_t smem = StreamCfg<CODEC, LW>::kSmemBytes;
  auto kernel = qlinear_stream_kernel<CODEC, LW>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kernel<<<(unsigned)grid, StreamRoles<LW>::kThreads, smem, stream>>>(args);
  return cudaGetLastError();
}

}  // namespace

size_t stream_weight_bytes(int codec, int64_t rows_padded, int64_t columns) {
  return (size_t)(rows_padded / kTileRows) * (size_t)(columns / 32) * (size_t)kTileRows * ((codec == 2 ? 16 : 32) + 2);
}

cudaError_t launch_repack_stream(const TiledWeight& w, const RepackParts& parts, cudaStream_t stream) {
  const int64_t kblocks = w.columns / 32;
  const int64_t total = w.rows_padded * kblocks;
  if (total == 0) return cudaSuccess;
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 32);
  repack_stream_kernel<<<grid, 256, 0, stream>>>(parts, w.codec, w.rows, w.rows_padded, kblocks, w.interleave8, w.quants);
  return cudaGetLastError();
}

StreamPlan plan_stream(const TiledWeight& w, int64_t vectors, int sm_count) {
  StreamPlan p;
  const int64_t chunk = std::min<int64_t>(vectors, kStreamMaxVectors);
  p.nvp = (int)((chunk + 31) / 32 * 32);
  p.tiles = (int)(w.rows_padded / kTileRows);
  p.spt = (int)(w.columns / (32 * kStageBlocks));
  p.total_units = p.tiles * p.spt;
  const int ctas = std::max(1, std::min(sm_count, p.total_units));
  int per = (p.total_units + ctas - 1) / ctas;
  per = std::max(per, std::min(p.spt, 4));  // a CTA's set-up is worth a few stages
  p.units_per_cta = per;
  p.grid = (p.total_units + per - 1) / per;
  const int two_per_cta = 2 * p.grid, diagonal = p.grid + p.tiles - 1;
  p.slot_mode = diagonal < two_per_cta ? 1 : 0;
  const int slots = per % p.spt == 0 ? 0 : std::min(two_per_cta, diagonal);  // whole tiles per CTA: nothing is partial
  p.own_sum = (p.spt + per - 1) / per + 1 <= kOwnSumMaxRanges ? 1 : 0;  // most ranges a tile can be cut into
  p.xh_bytes = (size_t)(w.columns / 8) * p.nvp * 16;
  p.partial_bytes = (size_t)slots * p.nvp * kTileRows * sizeof(float);
  return p;
}

cudaError_t launch_qlinear_stream(const TiledWeight& w, const float* x, const __half* xh_ready, int64_t vectors, const float* bias,
                                  const float* residual, int epilogue, float* out, __half* out_xh, __half* xh, float* partials,
                                  DeviceStatus* status, int sm_count, cudaStream_t stream, int* launches) {
  const int out_cols = (int)(epilogue == ETC_EPILOGUE_SWIGLU ? w.rows / 2 : w.rows);
  const int K = (int)w.columns;
  for (int64_t v0 = 0; v0 < vectors; v0 += kStreamMaxVectors) {
    const int64_t chunk = std::min<int64_t>(kStreamMaxVectors, vectors - v0);
    const StreamPlan plan = plan_stream(w, chunk, sm_count);
    const bool ready = xh_ready != nullptr && vectors <= 32;  // producer already stored [K/8][32][8] f16
    if (!ready) {
      const int total = (K / 8) * plan.nvp;
      const unsigned cgrid = (unsigned)std::min((total + 255) / 256, 148 * 4);
      convert_xh8_rows_kernel<<<cgrid, 256, 0, stream>>>(x + v0 * K, (int)chunk, K, plan.nvp, xh);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      if (launches) ++*launches;
    }
    StreamArgs args;
    args.weights = w.quants;
    args.xh = ready ? xh_ready : xh;
    args.bias = bias;
    args.residual = residual ? residual + v0 * out_cols : nullptr;
    args.out = out ? out + v0 * out_cols : nullptr;
    args.out_xh = vectors <= 32 ? out_xh : nullptr;
    args.out_xh_nv = 32;
    args.partials = partials;
    args.counters = w.counters;
    args.status = &status->code;
    args.vectors = (int)chunk;
    args.nvp = plan.nvp;
    args.rows = (int)w.rows;
    args.tiles = plan.tiles;
    args.spt = plan.spt;
    args.total_units = plan.total_units;
    args.units_per_cta = plan.units_per_cta;
    args.epilogue = epilogue;
    args.slot_mode = plan.slot_mode;
    args.own_sum = plan.own_sum;
    cudaError_t e;
    if (plan.nvp <= 32) e = w.codec == 2 ? launch_stream_pass<2, 1>(args, plan.grid, stream) : launch_stream_pass<8, 1>(args, plan.grid, stream);
    else e = w.codec == 2 ? launch_stream_pass<2, 4>(args, plan.grid, stream) : launch_stream_pass<8, 4>(args, plan.grid, stream);
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
    if (!plan.own_sum && plan.partial_bytes > 0) {
      qlinear_stream_sum_kernel<<<dim3((unsigned)plan.tiles, (unsigned)(plan.nvp / 32)), 512, 0, stream>>>(args);
      const cudaError_t e2 = cudaGetLastError();
      if (e2 != cudaSuccess) return e2;
      if (launches) ++*launches;
    }
  }
  return cudaSuccess;
}

}  // namespace etc
