// Dequant matvec for small decode batches (up to 16 input vectors) on Q4_0 / Q8_0 weights.
//
//   out[v, r] = sum_k x[v, k] * deq(W[r, k])        (quantized_linear, crates/runtime-cpu/src/quantized.rs:419-499)
//
// Why a second kernel beside the tcgen05 one: one tcgen05.mma retires 128 weight rows x 16 columns in about 130 cycles
// whatever the number of vectors (measured: 131 cycles for every N <= 128 at 1965 MHz), which caps that kernel at 0.4 of
// what HBM delivers for Q4_0. The legacy tensor path (mma.sync m16n8k16: one instruction per 256 weights and 8
// vectors, 0.46 instructions per cycle per SM on the same physical pipe) needs a quarter of the pipe at 16 vectors and
// an eighth at 8, so there the work is bounded by the dequantisation instructions and by memory, not by the pipe. It
// reads the same 128-row tile layout, so a weight has one copy in HBM.
//
// Data flow per CTA (8 consumer warps + 1 copy warp; three CTAs per SM at 8 vectors, two at 16):
//   * the copy warp fills a ring of 3 or 4 stages in shared memory. A stage is one 128-row layout tile x 8 (Q4_0) or 4
//     (Q8_0) blocks of 32 columns: the packed weights [block][128 rows][16 or 32 B] and the scales [block][128] f16 are
//     each contiguous in the layout, so they arrive as two bulk copies (cp.async.bulk, completion counted in bytes on
//     the stage's mbarrier); the stage's activations (f16, hand-off layout [K/8][stride][8]) arrive as 16-byte cp.async
//     copies issued by all 32 lanes, which arrive on the same mbarrier when they land. Weights do not depend on the
//     previous kernel of the stream, so under programmatic dependent launch the first stage's weights are requested
//     before the grid dependency wait; the rest of the ring follows once that stage has landed, so that every CTA's
//     first stage is served ahead of everybody's second and the consumers start early.
//   * consumer warp w owns rows 16w..16w+15 of the tile for the whole K range of the CTA: nothing is summed across
//     warps. It fetches the packed words of two blocks with one ldmatrix.x4 (lane (g, t) receives word t of rows g and
//     g+8, which is exactly the A-fragment ownership of mma.m16n8k16), splices nibbles / bytes into f16 mantissas (one
//     three-input logic op or byte permute, then one hsub2 / hfma2 that removes the splice bias and the code offset; the
//     constants live in registers because the two-immediate forms cost an extra instruction each), reads the B
//     fragments of a block with 16-byte shared-memory loads (column groups padded so that the four t lanes hit
//     different banks) and issues two MMAs per block and 8 vectors. The integer codes go through the MMA unscaled; the
//     f32 block scale is applied to the block's partial sums (4 FFMA per 8 vectors). Inside a block, lane t owns logical
//     columns 8t..8t+7 (Q4_0) or 4t..4t+3 and 16+4t..16+4t+3 (Q8_0) on both operands, so no data moves between lanes.
//   * work is cut stream-K style: units (tile, stage) in tile-major order, an equal contiguous run per CTA. A run's
//     segment that covers its tile's whole K applies the epilogue straight from the accumulator registers (SwiGLU pairs
//     a gate row g with its up row g+8 inside one thread). Only the first and the last segment of a run can cover part
//     of a tile's K: the consumers store such partial sums and go on; the copy warp draws a ticket on the tile once the
//     piece is stored; at the end of its run a CTA that drew a tile's last ticket adds the tile's pieces in CTA order
//     (deterministic) and applies the epilogue. Nobody waits for another CTA.
// Every mbarrier wait is bounded; on expiry the abort flag is raised, all roles run their loops dry, the copy warp lets
// its copies land, and the status word reports 3. Tickets of tiles that were in flight at that moment may be left
// non-zero: weights that were used by a call that ended with that status must be rebuilt.
//
// Roofline: HBM. Algorithmic bytes = rows*K/32*{18,34} + activation and output bytes. Measured at 8 vectors, Q4_0:
// 0.61 of the copy bandwidth on [128256 x 4096], 0.41 on [28672 x 4096], 0.30 on [14336 x 4096] (where ramp-up and the
// last tickets are a third of the run); the steady state is bounded by instruction issue (about 33 instructions per
// 512 weights at 1.7 instructions per cycle per SM), not by the ring, which alone streams at 0.85-0.93.
#include <cuda_fp16.h>

#include <algorithm>

#include "chain.cuh"
#include "kernels.h"
#include "tc05.cuh"

namespace etc {

namespace {

using namespace tc05;

constexpr int kMvRows = 128;  // rows of a layout tile
constexpr int kMvConsumerWarps = 8;
constexpr int kMvConsumerThreads = kMvConsumerWarps * 32;
constexpr int kMvThreads = kMvConsumerThreads + 32;

template <int CODEC, int NT>
struct MvCfg {
  static constexpr int kNV = NT * 8;
  static_assert(NT == 1 || NT == 2, "one pass takes 8 or 16 vectors");
  static constexpr int kMT = 1;  // m16 tiles per warp
  static constexpr int kGroupTiles = kMT * (kMvConsumerWarps / 8);  // layout tiles per row group: 8 warps cover one tile's rows
  static constexpr int kGroupRows = kGroupTiles * kMvRows;
  static constexpr int kStageBlocks = CODEC == 2 ? 8 : 4;
  static constexpr int kCtasPerSm = NT == 1 ? 3 : 2;
  static constexpr int kStages = NT == 1 ? 3 : 4;
  static constexpr bool kScaleWeights = false;  // the f32 block scale is applied to the block's sums, not to the f16 weights
  static constexpr uint32_t kBlockQBytes = CODEC == 2 ? 2048 : 4096;
  static constexpr uint32_t kTileQBytes = kStageBlocks * kBlockQBytes;  // one layout tile's share of a stage
  static constexpr uint32_t kTileSBytes = kStageBlocks * 256;
  static constexpr uint32_t kStageQBytes = kGroupTiles * kTileQBytes;
  static constexpr uint32_t kStageSBytes = kGroupTiles * kTileSBytes;
  // activations of a stage: [4 * blocks column groups][kNV rows][8 halves], each group padded by 32 bytes so that the
  // 16-byte reads of lanes t = 0..3 (consecutive groups) and g, g+1 (consecutive rows) fall into different banks
  static constexpr uint32_t kGroupBytes = kNV * 16 + 32;
  static constexpr uint32_t kStageXBytes = kStageBlocks * 4 * kGroupBytes;
  static constexpr uint32_t kStageBytes = kStageQBytes + kStageSBytes + kStageXBytes;
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + (2 * kStages + 4) * sizeof(uint64_t) + 16;
  static_assert(CODEC != 2 || kStageBlocks % 2 == 0, "Q4_0 fetches two blocks per ldmatrix");
  static_assert(kStageBytes % 16 == 0 && kTileQBytes % 16 == 0, "bulk copies need 16-byte alignment");
  static_assert(kSmemBytes <= (kCtasPerSm == 3 ? 75 : 113) * 1024, "CTAs per SM");
};

struct MvArgs {
  const unsigned char* quants;  // [tile][kblock][128 rows][16 B (Q4_0) | 32 B (Q8_0)]
  const __half* scales;         // [tile][kblock][128]
  const __half* xh;             // f16 [K/8][xh_nv][8], rows >= vectors are zero
  int xh_nv;
  const float* bias;
  const float* residual;
  float* out;
  __half* out_xh;               // optional f16 copy of the result in the hand-off layout [cols/8][out_xh_nv][8]
  int out_xh_nv;
  float* partials;              // [grid][2][NT*8][group rows] f32
  int* tickets;                 // [row groups], zero between launches
  unsigned long long* status;
  int vectors, rows, tiles, kblocks, spt, units, upc, epilogue;
  // Splice constants, passed as arguments so that they live in (uniform) registers: with literals the compiler emits
  // two-immediate forms that cost an extra instruction each (a three-input logic op or an f16x2 fma takes one immediate).
  uint32_t c_magic, c_bias_lo, c_sixteenth, c_bias_hi, c_bias_q8, c_perm_fill;
};


__device__ __forceinline__ void ldmatrix_x4(const void* smem_row, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(smem_row)) : "memory");
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
// This thread's earlier cp.async copies arrive on the mbarrier when they have landed (counted in the barrier's
// expected arrivals, not added to them).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct SpliceConsts {
  uint32_t magic;      // half2(1024, 1024): a nibble spliced into the mantissa reads 1024 + code
  uint32_t bias_lo;    // half2(1032, 1032) = 1024 + 8
  uint32_t sixteenth;  // half2(1/16, 1/16)
  uint32_t bias_hi;    // half2(-72, -72) = -(1024 / 16 + 8)
  uint32_t bias_q8;    // half2(1152, 1152) = 1024 + 128
  uint32_t perm_fill;  // 0x64646464: the exponent byte of 1024 for the byte splice
};
__device__ __forceinline__ uint32_t and_or(uint32_t x, uint32_t mask, uint32_t fill) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(x), "r"(mask), "r"(fill));  // (x & mask) | fill
  return d;
}
__device__ __forceinline__ uint32_t sub_h2(uint32_t x, uint32_t y) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(x), "r"(y));
  return d;
}
__device__ __forceinline__ uint32_t fma_h2(uint32_t x, uint32_t y, uint32_t z) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(y), "r"(z));
  return d;
}
// One packed Q4_0 word (8 nibbles, logical column j of the word at bit {0,16,8,24,4,20,12,28}[j]) -> the integers
// code - 8 as four half2 in column order: (c0,c1) (c2,c3) for the block's first MMA, (c4,c5) (c6,c7) for the second.
__device__ __forceinline__ void q4_codes(uint32_t q, const SpliceConsts& k, uint32_t (&o)[4]) {
  const uint32_t qs = q >> 8;
  o[0] = sub_h2(and_or(q, 0x000F000Fu, k.magic), k.bias_lo);
  o[1] = sub_h2(and_or(qs, 0x000F000Fu, k.magic), k.bias_lo);
  o[2] = fma_h2(and_or(q, 0x00F000F0u, k.magic), k.sixteenth, k.bias_hi);
  o[3] = fma_h2(and_or(qs, 0x00F000F0u, k.magic), k.sixteenth, k.bias_hi);
}
// Four int8 -> (b0,b1) (b2,b3) as half2 integers.
__device__ __forceinline__ void q8_codes(uint32_t w, const SpliceConsts& k, uint32_t (&o)[2]) {
  const uint32_t x = w ^ 0x80808080u;
  o[0] = sub_h2(__byte_perm(x, k.perm_fill, 0x4140), k.bias_q8);
  o[1] = sub_h2(__byte_perm(x, k.perm_fill, 0x4342), k.bias_q8);
}

// One m16 tile x one block: a1 / a2 are the A fragments of the block's two MMAs (rows g, g+8 interleaved as the
// instruction wants them), sg / sg8 the block scales of the two rows.
template <int NT, bool SCALE_W>
__device__ __forceinline__ void tile_block(float (&acc)[NT][4], uint32_t (&a1)[4], uint32_t (&a2)[4], __half sg, __half sg8,
                                           const uint32_t (&b)[NT][4]) {
  if (SCALE_W) {
    const __half2 s = __half2half2(sg), s8 = __half2half2(sg8);
    a1[0] = h2u(__hmul2(u2h(a1[0]), s)); a1[2] = h2u(__hmul2(u2h(a1[2]), s));
    a2[0] = h2u(__hmul2(u2h(a2[0]), s)); a2[2] = h2u(__hmul2(u2h(a2[2]), s));
    a1[1] = h2u(__hmul2(u2h(a1[1]), s8)); a1[3] = h2u(__hmul2(u2h(a1[3]), s8));
    a2[1] = h2u(__hmul2(u2h(a2[1]), s8)); a2[3] = h2u(__hmul2(u2h(a2[3]), s8));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      mma_16816(acc[nt], a1[0], a1[1], a1[2], a1[3], b[nt][0], b[nt][1]);
      mma_16816(acc[nt], a2[0], a2[1], a2[2], a2[3], b[nt][2], b[nt][3]);
    }
  } else {
    const float fs = __half2float(sg), fs8 = __half2float(sg8);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float blk[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      mma_16816(blk, a1[0], a1[1], a1[2], a1[3], b[nt][0], b[nt][1]);
      mma_16816(blk, a2[0], a2[1], a2[2], a2[3], b[nt][2], b[nt][3]);
      acc[nt][0] = fmaf(fs, blk[0], acc[nt][0]);
      acc[nt][1] = fmaf(fs, blk[1], acc[nt][1]);
      acc[nt][2] = fmaf(fs8, blk[2], acc[nt][2]);
      acc[nt][3] = fmaf(fs8, blk[3], acc[nt][3]);
    }
  }
}

// Epilogue of one warp's accumulators of one layout tile: acc[nt] = {(row g, vector 2t), (row g, 2t+1), (row g+8, 2t),
// (row g+8, 2t+1)} of the m16 tile that starts at row `wr` of the tile. Loads (bias, residual) are issued for every element before the
// first store so that their latency is paid once.
template <int NT>
__device__ __forceinline__ void store_rows(const MvArgs& a, int tile, int wr, int g, int t, const float (&acc)[NT][4]) {
  const int R0 = tile * kMvRows + wr + g;  // row of elements 0 and 1; elements 2 and 3 sit 8 rows below
  float extra[NT][4];
  {
    const float b_lo = a.bias && R0 < a.rows ? a.bias[R0] : 0.0f;
    const float b_hi = a.bias && R0 + 8 < a.rows ? a.bias[R0 + 8] : 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int v = nt * 8 + 2 * t + (e & 1), R = R0 + (e >> 1) * 8;
        float x = e < 2 ? b_lo : b_hi;
        if (a.epilogue == ETC_EPILOGUE_RESIDUAL && v < a.vectors && R < a.rows) x += a.residual[(size_t)v * a.rows + R];
        extra[nt][e] = x;
      }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    if (a.epilogue == ETC_EPILOGUE_SWIGLU) {
      // rows are interleaved in groups of 8: row R0 (a gate row) pairs with row R0 + 8 (its up row)
      const int out_cols = a.rows >> 1;
      const int oc = (R0 >> 4) * 8 + (R0 & 7);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int v = nt * 8 + 2 * t + e;
        if (v >= a.vectors || R0 + 8 >= a.rows) continue;
        const float act = silu_tanh(acc[nt][e] + extra[nt][e]) * (acc[nt][2 + e] + extra[nt][2 + e]);
        if (a.out) a.out[(size_t)v * out_cols + oc] = act;
        if (a.out_xh)
          a.out_xh[((size_t)(oc >> 3) * a.out_xh_nv + v) * 8 + (oc & 7)] = __float2half_rn(fminf(fmaxf(act, -65504.f), 65504.f));
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int v = nt * 8 + 2 * t + (e & 1), R = R0 + (e >> 1) * 8;
        if (v >= a.vectors || R >= a.rows) continue;
        const float val = acc[nt][e] + extra[nt][e];
        if (a.out) a.out[(size_t)v * a.rows + R] = val;
        if (a.out_xh)
          a.out_xh[((size_t)(R >> 3) * a.out_xh_nv + v) * 8 + (R & 7)] = __float2half_rn(fminf(fmaxf(val, -65504.f), 65504.f));
      }
    }
  }
}

template <int CODEC, int NT>
__global__ void __launch_bounds__(kMvThreads, (MvCfg<CODEC, NT>::kCtasPerSm)) qlinear_mv_kernel(MvArgs a) {
  using Cfg = MvCfg<CODEC, NT>;
  constexpr int KS = Cfg::kStageBlocks, STAGES = Cfg::kStages, MT = Cfg::kMT, NV = Cfg::kNV, GR = Cfg::kGroupRows, TG = Cfg::kGroupTiles;
  constexpr uint32_t GS = Cfg::kGroupBytes;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* ring = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * Cfg::kStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* first_weights = empty + STAGES;  // the first stage's weight copies complete here (see the copy warp)
  uint64_t* piece_done = first_weights + 1;  // [2]: the consumers' partial sums of the run's first / last segment are stored
  uint64_t* tickets_done = piece_done + 2;   // the copy warp has taken the tickets of every stored piece
  volatile int* flags = reinterpret_cast<volatile int*>(tickets_done + 1);  // [0] abort, [1], [2] tickets of the two pieces

  chain_release();  // the next kernel of the stream may be scheduled; it waits for this one before touching its data
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int u0 = blockIdx.x * a.upc;
  const int u1 = min(a.units, u0 + a.upc);
  // A run covers the tail of its first group, whole groups, and the head of its last group. Only the first and the last
  // segment can cover part of a group's K ("pieces"): piece 0 = first segment, piece 1 = last segment of a later group.
  const int group_first = u0 / a.spt, st_first = u0 - group_first * a.spt;
  const int group_last = (u1 - 1) / a.spt, st_last = (u1 - 1) - group_last * a.spt;
  const bool piece0 = st_first != 0 || (group_last == group_first && st_last != a.spt - 1);
  const bool piece1 = group_last != group_first && st_last != a.spt - 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1 + 32);  // the weight copies' expect_tx arrival + one arrival per lane's activation copies
      mbar_init(&empty[s], kMvConsumerWarps);
    }
    mbar_init(first_weights, 1);
    mbar_init(&piece_done[0], kMvConsumerWarps);
    mbar_init(&piece_done[1], kMvConsumerWarps);
    mbar_init(tickets_done, 1);
    flags[0] = 0;
    flags[1] = -1;
    flags[2] = -1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == kMvConsumerWarps) {
    // ------------------------------------------------------------------ copy warp
    const int n = u1 - u0;
    auto issue_weights = [&](int i, uint64_t* bar) {  // one lane: the bulk copies of unit u0 + i, completing on `bar`
      const int u = u0 + i, s = i % STAGES;
      const int group = u / a.spt, st = u - group * a.spt;
      const int kb = st * KS;
      const int valid = min(KS, a.kblocks - kb);
      const int tiles_here = min(TG, a.tiles - group * TG);
      unsigned char* dst = ring + (size_t)s * Cfg::kStageBytes;
      mbar_arrive_expect_tx(bar, (uint32_t)(tiles_here * valid) * (Cfg::kBlockQBytes + 256u));
      for (int m = 0; m < tiles_here; ++m) {
        const size_t block_index = (size_t)(group * TG + m) * a.kblocks + kb;
        bulk_copy_g2s(dst + (size_t)m * Cfg::kTileQBytes, a.quants + block_index * Cfg::kBlockQBytes, (uint32_t)valid * Cfg::kBlockQBytes, bar);
        bulk_copy_g2s(dst + Cfg::kStageQBytes + (size_t)m * Cfg::kTileSBytes, a.scales + block_index * kMvRows, (uint32_t)valid * 256u, bar);
      }
    };
    // Tickets (one lane): once the consumers have stored a piece, count this CTA in on the piece's group. The outcome
    // goes to flags[1 + k]; whoever draws the last ticket of a group adds its pieces up at the end of its run.
    bool ticket_pending[2] = {piece0, piece1};
    auto take_ticket = [&](int k, bool blocking) {
      if (!ticket_pending[k]) return;
      if (blocking ? !mbar_wait_relaxed(&piece_done[k], 0, flags, 64) : !mbar_try_wait(&piece_done[k], 0)) return;
      ticket_pending[k] = false;
      if (flags[0]) return;
      __threadfence();
      const int ticket = atomicAdd(&a.tickets[k == 0 ? group_first : group_last], 1);
      __threadfence();
      flags[1 + k] = ticket;
    };
    // Weights do not depend on the stream's previous kernel: the first stage starts before the grid dependency wait.
    // The other stages of the ring are issued once the first one has landed, so that every CTA's first stage is served
    // ahead of everybody's second and the consumers start while the rest of the ring is still in flight.
    int weights_issued = 0;
    if (lane == 0) {
      issue_weights(0, first_weights);
      weights_issued = 1;
    }
    chain_wait();
    int st = st_first;
    for (int i = 0; i < n; ++i) {
      const int s = i % STAGES;
      if (i >= STAGES) {
        const uint32_t round = (uint32_t)(i / STAGES);
        const bool ok = mbar_wait_relaxed(&empty[s], (round & 1) ^ 1, flags, 32);
        if (!__all_sync(0xffffffffu, ok)) break;
        if (lane == 0) {
          issue_weights(i, &full[s]);
          weights_issued = i + 1;
        }
      }
      // the stage's activations: column groups [kb*4, (kb + valid)*4) x rows [0, NV) of the hand-off layout
      const int kb = st * KS;
      const int valid = min(KS, a.kblocks - kb);
      unsigned char* xdst = ring + (size_t)s * Cfg::kStageBytes + Cfg::kStageQBytes + Cfg::kStageSBytes;
      const __half* xsrc = a.xh + (size_t)kb * 4 * a.xh_nv * 8;
      for (int c = lane; c < valid * 4 * NV; c += 32) {
        const int grp = c / NV, row = c - grp * NV;
        cp_async_16(xdst + (size_t)grp * GS + row * 16, xsrc + ((size_t)grp * a.xh_nv + row) * 8);
      }
      cp_async_arrive(&full[s]);
      if (lane == 0) {
        if (i == 0) {
          if (mbar_wait_relaxed(first_weights, 0, flags, 32)) mbar_arrive(&full[0]);  // stands in for the copies' own arrival
          for (int j = 1; j < min(STAGES, n); ++j) issue_weights(j, &full[j]);
          weights_issued = min(STAGES, n);
        }
        take_ticket(0, false);
      }
      if (++st == a.spt) st = 0;
    }
    cp_async_wait_all();
    if (lane == 0) {
      take_ticket(0, true);
      take_ticket(1, true);
      mbar_arrive(tickets_done);
      if (flags[0]) {
        // give-up path: this warp's own bulk copies must have landed (bounded) before the CTA's shared memory goes away
        for (unsigned spin = 0; spin < (1u << 20) && !mbar_try_wait(first_weights, 0); ++spin) __nanosleep(64);
        for (int i = max(1, weights_issued - STAGES); i < weights_issued; ++i) {
          const uint32_t parity = (uint32_t)(i / STAGES) & 1;
          for (unsigned spin = 0; spin < (1u << 20) && !mbar_try_wait(&full[i % STAGES], parity); ++spin) __nanosleep(64);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumer warps
    const int g = lane >> 2, t = lane & 3;
    const int wt = (warp >> 3) * MT;  // this warp's first layout tile inside the group
    const int wr = (warp & 7) * 16;   // its first row inside each of its layout tiles
    const SpliceConsts kc = {a.c_magic, a.c_bias_lo, a.c_sixteenth, a.c_bias_hi, a.c_bias_q8, a.c_perm_fill};
    float acc[MT][NT][4];
    bool alive = true;

    chain_wait();  // outputs, partials and tickets belong to the stream's earlier kernels until here
    int group = group_first, st = st_first;
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[m][nt][e] = 0.0f;
    for (int u = u0; u < u1; ++u) {
      const int i = u - u0, s = i % STAGES;
      const uint32_t parity = (uint32_t)(i / STAGES) & 1;
      const int valid = min(KS, a.kblocks - st * KS);
      if (alive) alive = mbar_wait_warp(&full[s], parity, flags);
      const unsigned char* stage_q = ring + (size_t)s * Cfg::kStageBytes;
      const __half* stage_s = reinterpret_cast<const __half*>(stage_q + Cfg::kStageQBytes);
      const unsigned char* stage_x = stage_q + Cfg::kStageQBytes + Cfg::kStageSBytes;
      if (alive) {
        if (CODEC == 2) {
#pragma unroll
          for (int kbl = 0; kbl < KS; kbl += 2) {
            if (kbl >= valid) break;  // block counts are even: a pair is valid or not as a whole
            // packed words of blocks kbl and kbl+1: rows g / g+8 of this warp's m16 tile, word t
            uint32_t w[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const unsigned char* q0 = stage_q + (size_t)(wt + m) * Cfg::kTileQBytes + (size_t)kbl * 2048 + (size_t)wr * 16;
              ldmatrix_x4(q0 + (size_t)(lane >> 4) * 2048 + (size_t)(lane & 15) * 16, w[m][0], w[m][1], w[m][2], w[m][3]);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // B fragments of the block: {MMA1.b0, MMA1.b1, MMA2.b0, MMA2.b1} of vector nt*8 + g
              uint32_t b[NT][4];
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const uint4 v = *reinterpret_cast<const uint4*>(stage_x + (size_t)((kbl + h) * 4 + t) * GS + (nt * 8 + g) * 16);
                b[nt][0] = v.x; b[nt][1] = v.y; b[nt][2] = v.z; b[nt][3] = v.w;
              }
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const __half* sc = stage_s + (size_t)(wt + m) * (Cfg::kTileSBytes / 2) + (kbl + h) * kMvRows + wr + g;
                uint32_t cg[4], cg8[4];
                q4_codes(w[m][2 * h], kc, cg);
                q4_codes(w[m][2 * h + 1], kc, cg8);
                uint32_t a1[4] = {cg[0], cg8[0], cg[1], cg8[1]};
                uint32_t a2[4] = {cg[2], cg8[2], cg[3], cg8[3]};
                tile_block<NT, Cfg::kScaleWeights>(acc[m], a1, a2, sc[0], sc[8], b);
              }
            }
          }
        } else {
#pragma unroll
          for (int kbl = 0; kbl < KS; ++kbl) {
            if (kbl >= valid) break;
            uint32_t b[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const unsigned char* p = stage_x + (size_t)(kbl * 4 + (t >> 1)) * GS + (nt * 8 + g) * 16 + (t & 1) * 8;
              const uint2 v0 = *reinterpret_cast<const uint2*>(p);
              const uint2 v1 = *reinterpret_cast<const uint2*>(p + 2 * GS);
              b[nt][0] = v0.x; b[nt][1] = v0.y; b[nt][2] = v1.x; b[nt][3] = v1.y;
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              // matrices: rows 0-7 / 8-15 of bytes 0-15 (columns 4t..4t+3), then rows 0-7 / 8-15 of bytes 16-31
              const int mi = lane >> 3, rr = lane & 7;
              const unsigned char* q0 = stage_q + (size_t)(wt + m) * Cfg::kTileQBytes + (size_t)kbl * 4096 + (size_t)wr * 32;
              uint32_t w0, w1, w2, w3;
              ldmatrix_x4(q0 + (size_t)((mi & 1) * 8 + rr) * 32 + (mi >> 1) * 16, w0, w1, w2, w3);
              uint32_t lg[2], lg8[2], hg[2], hg8[2];
              q8_codes(w0, kc, lg);
              q8_codes(w1, kc, lg8);
              q8_codes(w2, kc, hg);
              q8_codes(w3, kc, hg8);
              uint32_t a1[4] = {lg[0], lg8[0], lg[1], lg8[1]};
              uint32_t a2[4] = {hg[0], hg8[0], hg[1], hg8[1]};
              const __half* sc = stage_s + (size_t)(wt + m) * (Cfg::kTileSBytes / 2) + kbl * kMvRows + wr + g;
              tile_block<NT, Cfg::kScaleWeights>(acc[m], a1, a2, sc[0], sc[8], b);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);

      if (u + 1 == u1 || st + 1 == a.spt) {
        // ---------------------------------------------------------------- end of a group segment
        const bool is_piece = (group == group_first && piece0) || (group == group_last && group != group_first && piece1);
        if (!is_piece) {
          if (!flags[0]) {
#pragma unroll
            for (int m = 0; m < MT; ++m) store_rows<NT>(a, group * TG + wt + m, wr, g, t, acc[m]);
          }
        } else {
          // this thread's elements of the piece, [vector][row of the group]; the copy warp takes the ticket
          const int k = group == group_first ? 0 : 1;
          float* piece = a.partials + ((size_t)blockIdx.x * 2 + (k == 0 && st_first != 0 ? 0 : 1)) * NV * GR;
#pragma unroll
          for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e)
                piece[(size_t)(nt * 8 + 2 * t + (e & 1)) * GR + (wt + m) * kMvRows + wr + g + (e >> 1) * 8] = acc[m][nt][e];
          __syncwarp();
          if (lane == 0) mbar_arrive(&piece_done[k]);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][nt][e] = 0.0f;
      }
      if (++st == a.spt) { st = 0; ++group; }
    }
    // ---------------------------------------------------------------- groups this CTA drew the last ticket of
    if (piece0 || piece1) {
      if (alive) alive = mbar_wait_warp(tickets_done, 0, flags);
      for (int k = 0; k < 2; ++k) {
        if (!(k == 0 ? piece0 : piece1) || !alive || flags[0]) continue;
        const int grp = k == 0 ? group_first : group_last;
        const int first_unit = grp * a.spt;
        const int c_first = first_unit / a.upc;
        const int c_last = (first_unit + a.spt - 1) / a.upc;
        if (flags[1 + k] != c_last - c_first) continue;  // another CTA arrives later and finishes the group
        if (threadIdx.x == 0) a.tickets[grp] = 0;          // ready for the next launch
        __threadfence();
        // CTA order (the same sum whoever arrives last); a tile's loads of one piece are issued before its adds
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float sum[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) sum[nt][e] = 0.0f;
          for (int c = c_first; c <= c_last; ++c) {
            const float* src = a.partials + ((size_t)c * 2 + (c * a.upc > first_unit ? 0 : 1)) * NV * GR;
            float p[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e)
                p[nt][e] = __ldcg(src + (size_t)(nt * 8 + 2 * t + (e & 1)) * GR + (wt + m) * kMvRows + wr + g + (e >> 1) * 8);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e) sum[nt][e] += p[nt][e];
          }
          store_rows<NT>(a, grp * TG + wt + m, wr, g, t, sum);
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && flags[0]) atomicCAS(a.status, 0ull, 3ull);  // a bounded wait expired
}

// f32 [vectors, K] -> f16 [K/8][NV][8] (rows >= vectors are zero), saturating at the f16 range.
template <int NV>
__global__ void mv_convert_kernel(const float* __restrict__ x, int vectors, int K, __half* __restrict__ xh) {
  chain_release();
  chain_wait();
  const int total = (K / 8) * NV;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int kg = idx / NV, n = idx - kg * NV;
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (n < vectors) {
      const float4 lo = *reinterpret_cast<const float4*>(x + (size_t)n * K + kg * 8);
      const float4 hi = *reinterpret_cast<const float4*>(x + (size_t)n * K + kg * 8 + 4);
      auto sat = [](float v) { return fminf(fmaxf(v, -65504.f), 65504.f); };
      packed.x = h2u(__floats2half2_rn(sat(lo.x), sat(lo.y)));
      packed.y = h2u(__floats2half2_rn(sat(lo.z), sat(lo.w)));
      packed.z = h2u(__floats2half2_rn(sat(hi.x), sat(hi.y)));
      packed.w = h2u(__floats2half2_rn(sat(hi.z), sat(hi.w)));
    }
    reinterpret_cast<uint4*>(xh)[idx] = packed;
  }
}

template <int CODEC, int NT>
cudaError_t launch_mv_pass(const MvArgs& args, int grid, cudaStream_t stream) {
  constexpr size_t smem = MvCfg<CODEC, NT>::kSmemBytes;
  auto kernel = qlinear_mv_kernel<CODEC, NT>;
  const cudaError_t attr = opt_in_shared_memory(kernel, smem);
  if (attr != cudaSuccess) return attr;
  return launch_chained(kernel, dim3((unsigned)grid), dim3((unsigned)kMvThreads), smem, stream, args);
}

size_t mv_xh_region(int nt, int64_t columns) { return ((size_t)(columns / 8) * nt * 8 * 16 + 255) & ~(size_t)255; }

}  // namespace

// Measured on a B200 (Q4_0 and Q8_0, rows x K from 4096 x 4096 to 128256 x 4096): the matvec kernel is ahead of the tcgen05
// kernel up to 16 vectors (1.1x to 1.4x on the large shapes) and behind it at 32, where both paths are bound by the one
// tensor pipe and the tcgen05 kernel's per-weight instruction count is lower.
int mv_max_vectors() { return 16; }

MvPlan plan_mv(const TiledWeight& w, int64_t vectors, int sm_count) {
  MvPlan p;
  p.nt = vectors <= 8 ? 1 : 2;  // one pass takes up to 16 vectors
  const int mt = kMvConsumerWarps / 8;  // layout tiles per row group
  const int ks = w.codec == 2 ? 8 : 4;
  const int kblocks = (int)(w.columns / 32);
  p.tiles = (int)(w.rows_padded / kMvRows);
  p.groups = (p.tiles + mt - 1) / mt;
  p.spt = (kblocks + ks - 1) / ks;
  p.units = p.groups * p.spt;
  const int target = std::max(1, sm_count) * (p.nt == 1 ? 3 : 2);  // resident CTAs: three per SM at 8 vectors, else two
  p.upc = std::max((p.units + target - 1) / target, std::min(2, p.spt));  // at least two stages per CTA
  p.grid = (p.units + p.upc - 1) / p.upc;
  p.xh_bytes = mv_xh_region(p.nt, w.columns);
  p.partial_bytes = (size_t)p.grid * 2 * p.nt * 8 * mt * kMvRows * sizeof(float);
  return p;
}

cudaError_t launch_qlinear_mv(const TiledWeight& w, const float* x, const __half* xh_ready, int64_t vectors, const float* bias,
                              const float* residual, int epilogue, float* out, __half* out_xh, void* scratch,
                              DeviceStatus* status, int sm_count, cudaStream_t stream, int* launches, int xh_nv) {
  if (!w.counters) return cudaErrorInvalidValue;
  const int out_cols = (int)(epilogue == ETC_EPILOGUE_SWIGLU ? w.rows / 2 : w.rows);
  const int K = (int)w.columns;
  for (int64_t v0 = 0; v0 < vectors; v0 += 16) {
    const int64_t chunk = std::min<int64_t>(16, vectors - v0);
    const MvPlan plan = plan_mv(w, chunk, sm_count);
    const int nv = plan.nt * 8;
    const bool single = vectors <= 16;  // the hand-off layouts hold one pass
    MvArgs a;
    a.quants = w.quants;
    a.scales = w.scales;
    __half* xh_scratch = reinterpret_cast<__half*>(scratch);
    if (single && xh_ready && nv <= xh_nv) {  // the producer kernel already stored the f16 layout
      a.xh = xh_ready;
      a.xh_nv = xh_nv;
    } else {
      if (!x) return cudaErrorInvalidValue;
      const int total = (K / 8) * nv;
      const unsigned cgrid = (unsigned)std::min((total + 255) / 256, 148 * 2);
      const float* xin = x + v0 * w.columns;
      cudaError_t ce;
      if (plan.nt == 1) ce = launch_chained(mv_convert_kernel<8>, dim3(cgrid), dim3(256), 0, stream, xin, (int)chunk, K, xh_scratch);
      else ce = launch_chained(mv_convert_kernel<16>, dim3(cgrid), dim3(256), 0, stream, xin, (int)chunk, K, xh_scratch);
      if (ce != cudaSuccess) return ce;
      if (launches) ++*launches;
      a.xh = xh_scratch;
      a.xh_nv = nv;
    }
    a.bias = bias;
    a.residual = residual ? residual + v0 * out_cols : nullptr;
    a.out = out ? out + v0 * out_cols : nullptr;
    a.out_xh = single && vectors <= xh_nv ? out_xh : nullptr;
    a.out_xh_nv = xh_nv;
    a.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + plan.xh_bytes);
    a.tickets = w.counters;
    a.status = &status->code;
    a.vectors = (int)chunk;
    a.rows = (int)w.rows;
    a.tiles = plan.tiles;
    a.kblocks = K / 32;
    a.spt = plan.spt;
    a.units = plan.units;
    a.upc = plan.upc;
    a.epilogue = epilogue;
    a.c_magic = 0x64006400u;
    a.c_bias_lo = 0x64086408u;    // 1032 = 0x6408
    a.c_sixteenth = 0x2C002C00u;  // 1/16 = 0x2C00
    a.c_bias_hi = 0xD480D480u;    // -72 = 0xD480
    a.c_bias_q8 = 0x64806480u;    // 1152 = 0x6480
    a.c_perm_fill = 0x64646464u;
    cudaError_t e;
    const bool q4 = w.codec == 2;
    if (plan.nt == 1) e = q4 ? launch_mv_pass<2, 1>(a, plan.grid, stream) : launch_mv_pass<8, 1>(a, plan.grid, stream);
    else e = q4 ? launch_mv_pass<2, 2>(a, plan.grid, stream) : launch_mv_pass<8, 2>(a, plan.grid, stream);
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

}  // namespace etc
