// Dequant linear on the 5th-generation tensor cores (tcgen05) for Q4_0 / Q8_0 weights.
//
//   out[v, r] = sum_k x[v, k] * deq(W[r, k])        (quantized_linear, crates/runtime-cpu/src/quantized.rs:419-499)
//
// Mapping onto tcgen05.mma.cta_group::1.kind::f16 (M = 128, N = NV, K = 16 per instruction):
//   * A operand = 128 weight rows, read from TENSOR MEMORY. Four "dequant" warps own one TMEM lane
//     (= one weight row) per thread: a thread streams its row's packed blocks from HBM (16-byte coalesced
//     loads, prefetched in registers), expands nibbles/bytes to f16 in registers, multiplies by the block
//     scale and writes 16 columns per 32-value block with tcgen05.st. Weights never touch shared memory.
//   * B operand = the NV input vectors (activations), f16 in shared memory in the canonical K-major
//     no-swizzle layout: 8-column groups of [NV rows][8 halves] (16 bytes per row), which is exactly how
//     the producer stores activations in global memory ("xh8": [K/8][NV][8] f16), so a stage of 128
//     columns is ONE contiguous cp.async.bulk copy completing on an mbarrier.
//   * D = f32 accumulator [128 x NV] in TMEM, read back once per CTA with tcgen05.ld.
// A CTA is 6 warps: 4 dequant/epilogue warps, 1 bulk-copy warp, 1 MMA-issue warp (one elected lane each).
// Stages of 4 blocks (128 columns) cycle through a ring of kStages TMEM A buffers + smem B buffers guarded
// by full_a / full_b / empty mbarriers; tcgen05.commit releases a stage when its MMAs have retired.
// Split-K over grid.y writes f32 partials that qlinear_reduce_kernel sums; with one split the epilogue
// (bias, residual add, SwiGLU over interleaved gate/up rows) runs straight from TMEM.
//
// Every mbarrier wait is bounded: on expiry the thread raises the abort flag and the status word, all
// roles fall through to the teardown, TMEM is freed and the kernel returns.
//
// Roofline: algorithmic bytes = rows*K/32*{18,34} + 2*NV*K + 4*V*rows. At NV <= 128 the kernel is bound by the rate at
// which an SM retires tcgen05.mma instructions: measured 131 cycles each at 1965 MHz for every N <= 128 (M = 64 or 128,
// A in tensor or shared memory, one to four accumulators), i.e. 2048 weights per 131 cycles = 0.39 of what HBM could
// feed for Q4_0; at NV = 256 (138 cycles) it is tensor-throughput bound.
#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "chain.cuh"
#include "codecs.cuh"
#include "kernels.h"
#include "tc05.cuh"

namespace etc {

namespace {

constexpr int kUmmaRows = 128;
constexpr int kDequantThreads = 128;  // one TMEM lane (weight row) per thread of a dequant group

// Pipeline shape: stages of four 32-value blocks in a ring of three (TMEM for the expanded weights, shared memory for
// the activations); for NV <= 64 two CTAs share an SM (256 TMEM columns each) and overlap each other's phases.
template <int NV>
struct UmmaCfg {
  static constexpr int kGroups = NV == 256 ? 2 : 1;  // at 256 vectors the MMAs of a stage take as long as one group needs to expand it
  static constexpr int kStageBlocks = 4;   // 32-value blocks per stage (K = 16 per MMA: 2 MMAs per block)
  static constexpr int kStages = 3;
  static constexpr int kAColsPerStage = kStageBlocks * 16;  // 32-bit TMEM columns holding the stage's f16 per lane
  static constexpr int kThreads = (4 * kGroups + 2) * 32;  // dequant warps + bulk-copy warp + MMA warp
  static constexpr uint32_t kStageBBytes = NV * kStageBlocks * 32 * 2;
  static constexpr uint32_t kTmemCols = NV + kStages * kAColsPerStage <= 256 ? 256 : 512;
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBBytes + (3 * kStages + 1) * sizeof(uint64_t) + 16;
};
constexpr int stage_blocks_for(int) { return 4; }
using namespace tc05;

struct UmmaArgs {
  const uint4* quants;    // Q4_0: [tile][kblock][128] uint4 ; Q8_0: [tile][kblock][128][2] uint4
  const __half* scales;   // [tile][kblock][128]
  const __half* xh;       // [K/8][NV][8] f16
  const float* bias;
  const float* residual;
  float* out;
  float* scratch;         // [splits][NV][rows_padded]
  unsigned long long* status;
  __half* out_xh;         // optional: result additionally stored as xh8 f16 [cols/8][out_xh_nv][8] for the next linear
  int out_xh_nv;
  int vectors, rows, rows_padded, kblocks, blocks_per_split, epilogue;
  int tile0;              // first row tile of this launch in the output (a segment of a weight fused from several codecs)
};

template <int CODEC, int NV>
__global__ void __launch_bounds__(UmmaCfg<NV>::kThreads) qlinear_umma_kernel(UmmaArgs a) {
  using Cfg = UmmaCfg<NV>;
  constexpr int kGroups = Cfg::kGroups, kStageBlocks = Cfg::kStageBlocks, kStages = Cfg::kStages;
  constexpr int kAColsPerStage = Cfg::kAColsPerStage;
  constexpr bool kNibbles = CODEC == 2 || CODEC == 12;      // 4-bit codes (Q4_0, re-cut Q4_K) or 8-bit (Q8_0, re-cut Q3_K / Q5_K / Q6_K)
  constexpr bool kPair = CODEC >= 12;                       // two f16 per (row, block): (scale, min) or the two half-block scales
  constexpr int QW = kNibbles ? 1 : 2;                      // uint4 words per (row, block)
  constexpr uint32_t kStageBBytes = Cfg::kStageBBytes;      // one stage of activations
  constexpr uint32_t kTmemCols = Cfg::kTmemCols;
  constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(NV >> 3) << 17) | ((uint32_t)(kUmmaRows >> 4) << 24);  // f16 x f16 -> f32
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* b_ring = smem;                                            // kStages * kStageBBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBBytes);
  uint64_t* full_a = bars;                // [kStages] 128 arrivals
  uint64_t* full_b = bars + kStages;      // [kStages] 1 arrival + tx bytes
  uint64_t* empty = bars + 2 * kStages;   // [kStages] 1 arrival (tcgen05.commit)
  uint64_t* done = bars + 3 * kStages;    // accumulator complete
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  chain_release();  // the next kernel (split-K sum or the step's next operator) may be scheduled already; it waits for this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  if (gridDim.z > 1) {  // this CTA's chunk of NV vectors: its activations, outputs and partials
    const size_t chunk = blockIdx.z;
    const size_t out_cols = a.epilogue == ETC_EPILOGUE_SWIGLU ? a.rows / 2 : a.rows;
    a.xh += chunk * ((size_t)a.kblocks * 4 * NV * 8);
    if (a.out) a.out += chunk * NV * out_cols;
    if (a.residual) a.residual += chunk * NV * out_cols;
    a.scratch += chunk * ((size_t)gridDim.y * NV * a.rows_padded);
    a.vectors = max(0, min(NV, a.vectors - (int)chunk * NV));
  }
  const int kb0 = split * a.blocks_per_split;
  const int kb1 = min(a.kblocks, kb0 + a.blocks_per_split);
  const int nstages = (kb1 - kb0 + kStageBlocks - 1) / kStageBlocks;

  // ---- dequant warps: group g = warp / 4 expands stages g, g + kGroups, ...; inside a group warp w owns TMEM lanes 32*(w%4)...
  const int group = warp >> 2;
  const int row = (warp & 3) * 32 + lane;  // TMEM lane == row inside the tile
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const uint4* qrow = a.quants + ((size_t)tile * a.kblocks) * (kUmmaRows * QW) + (size_t)row * QW;
  constexpr int SW = kPair ? 2 : 1;  // halves per (row, block) in the scale array
  const __half* srow = a.scales + (((size_t)tile * a.kblocks) * kUmmaRows + row) * SW;
  constexpr int PF = 2;  // of this group's stages, held packed in registers ahead of use
  uint4 qbuf[PF][kStageBlocks][QW];
  uint32_t sbuf[PF][kStageBlocks];  // one f16 (low half) or a pair
  auto load_stage = [&](int stage_index, int slot) {
#pragma unroll
    for (int b = 0; b < kStageBlocks; ++b) {
      const int kb = min(kb0 + stage_index * kStageBlocks + b, kb1 - 1);  // clamped: masked at use
#pragma unroll
      for (int w = 0; w < QW; ++w) qbuf[slot][b][w] = __ldg(qrow + (size_t)kb * (kUmmaRows * QW) + w);
      if (kPair) sbuf[slot][b] = __ldg(reinterpret_cast<const uint32_t*>(srow + (size_t)kb * kUmmaRows * 2));
      else sbuf[slot][b] = (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(srow + (size_t)kb * kUmmaRows));
    }
  };
  const int my_stages = nstages > group ? (nstages - group + kGroups - 1) / kGroups : 0;
  // the first packed stages are requested before tensor memory and the barriers are set up: weights depend on nothing
  if (warp < 4 * kGroups) {
#pragma unroll
    for (int p = 0; p < PF; ++p)
      if (p < my_stages) load_stage(group + p * kGroups, p);
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_a[s], kDequantThreads);
      mbar_init(&full_b[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(tmem_holder, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t d_tmem = tmem_base;             // columns [0, NV)
  const uint32_t a_tmem0 = tmem_base + NV;       // stage s at columns NV + s*kAColsPerStage

  if (warp < 4 * kGroups) {
    // ------------------------------------------------------------------ dequant warps
    bool ok = true;
    // Software pipeline: stage j is expanded in registers while the TMEM stores of stage j-1 are still in
    // flight; only then are those stores awaited and published, so the store latency hides behind ALU work.
    int pending_slot = -1;
    for (int j0 = 0; j0 < my_stages && ok; j0 += PF) {
#pragma unroll
      for (int p = 0; p < PF; ++p) {
        const int j = j0 + p;
        if (j >= my_stages || !ok) break;
        const int i = group + j * kGroups;  // global stage index
        const int s = i % kStages;
        const uint32_t round = (uint32_t)(i / kStages);
        const int valid = min(kStageBlocks, kb1 - (kb0 + i * kStageBlocks));
        uint32_t regs[kStageBlocks][16];
#pragma unroll
        for (int b = 0; b < kStageBlocks; ++b) {
          const uint32_t sraw = b < valid ? sbuf[p][b] : 0u;
          const __half2 pair = u2h(sraw);
          // first f16 of the entry: the block scale (codec 14: of values 0-15); second: the min (12, 13) or the scale of values 16-31 (14)
          const __half2 sc = __half2half2(__low2half(pair));
          const __half2 second = __half2half2(__high2half(pair));
          if (CODEC == 2) {
            const uint4 q = qbuf[p][b][0];
            expand_q4(q.x, sc, regs[b] + 0);
            expand_q4(q.y, sc, regs[b] + 4);
            expand_q4(q.z, sc, regs[b] + 8);
            expand_q4(q.w, sc, regs[b] + 12);
          } else if (CODEC == 12) {
            const uint4 q = qbuf[p][b][0];
            const __half2 neg_min = __hneg2(second);
            expand_q4k(q.x, sc, neg_min, regs[b] + 0);
            expand_q4k(q.y, sc, neg_min, regs[b] + 4);
            expand_q4k(q.z, sc, neg_min, regs[b] + 8);
            expand_q4k(q.w, sc, neg_min, regs[b] + 12);
          } else if (CODEC == 13) {
            const __half2 neg_min = __hneg2(second);
            const uint4 q0 = qbuf[p][b][0], q1 = qbuf[p][b][QW - 1];
            expand_q8k(q0.x, sc, neg_min, regs[b] + 0); expand_q8k(q0.y, sc, neg_min, regs[b] + 2);
            expand_q8k(q0.z, sc, neg_min, regs[b] + 4); expand_q8k(q0.w, sc, neg_min, regs[b] + 6);
            expand_q8k(q1.x, sc, neg_min, regs[b] + 8); expand_q8k(q1.y, sc, neg_min, regs[b] + 10);
            expand_q8k(q1.z, sc, neg_min, regs[b] + 12); expand_q8k(q1.w, sc, neg_min, regs[b] + 14);
          } else {
            const __half2 sc_hi = CODEC == 14 ? second : sc;
            const uint4 q0 = qbuf[p][b][0], q1 = qbuf[p][b][QW - 1];
            expand_q8(q0.x, sc, regs[b] + 0); expand_q8(q0.y, sc, regs[b] + 2); expand_q8(q0.z, sc, regs[b] + 4); expand_q8(q0.w, sc, regs[b] + 6);
            expand_q8(q1.x, sc_hi, regs[b] + 8); expand_q8(q1.y, sc_hi, regs[b] + 10); expand_q8(q1.z, sc_hi, regs[b] + 12); expand_q8(q1.w, sc_hi, regs[b] + 14);
          }
        }
        if (j + PF < my_stages) load_stage(group + (j + PF) * kGroups, p);  // refill this register slot
        if (pending_slot >= 0) {  // publish the previous stage of this group
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&full_a[pending_slot]);
        }
        // the MMAs that read this TMEM stage in the previous round must have retired
        ok = mbar_wait_warp(&empty[s], (round & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int b = 0; b < kStageBlocks; ++b)
          tmem_st16(a_tmem0 + lane_base + (uint32_t)(s * kAColsPerStage + b * 16), regs[b]);
        pending_slot = s;
      }
    }
    if (ok && pending_slot >= 0) {
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&full_a[pending_slot]);
    }
    // ------------------------------------------------------------------ epilogue (first group)
    if (group != 0) ok = false;
    if (ok) ok = mbar_wait(done, 0, abort_flag);
    chain_wait();  // outputs, residual and scratch may still be in use by the kernel before this one
    ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogue below shuffles across the warp
    if (ok) {
      tc_fence_after();
      const int r = (a.tile0 + tile) * kUmmaRows + row;
#pragma unroll 1
      for (int c0 = 0; c0 < NV; c0 += 32) {
        uint32_t acc[32];
        tmem_ld32(d_tmem + lane_base + (uint32_t)c0, acc);
        tmem_wait_ld();
        if (gridDim.y > 1) {
          float* dst = a.scratch + ((size_t)split * NV + c0) * a.rows_padded + r;
#pragma unroll
          for (int v = 0; v < 32; ++v) dst[(size_t)v * a.rows_padded] = __uint_as_float(acc[v]);
        } else if (a.epilogue == ETC_EPILOGUE_SWIGLU) {
          // rows are interleaved in groups of 8: lanes 0-7 of each 16 hold gate rows, lanes 8-15 their up rows
          const int oc = (r >> 4) * 8 + (r & 7);
          const float bias_v = a.bias && r < a.rows ? a.bias[r] : 0.0f;
#pragma unroll
          for (int v = 0; v < 32; ++v) {
            const float mine = __uint_as_float(acc[v]) + bias_v;
            const float partner = __shfl_xor_sync(0xffffffffu, mine, 8);
            if ((r & 8) == 0 && r + 8 < a.rows && c0 + v < a.vectors) {
              const float act = silu_tanh(mine) * partner;
              if (a.out) a.out[(size_t)(c0 + v) * (a.rows / 2) + oc] = act;
              if (a.out_xh)
                a.out_xh[((size_t)(oc >> 3) * a.out_xh_nv + (c0 + v)) * 8 + (oc & 7)] =
                    __float2half_rn(fminf(fmaxf(act, -65504.f), 65504.f));
            }
          }
        } else if (r < a.rows) {
          const float bias_v = a.bias ? a.bias[r] : 0.0f;
#pragma unroll
          for (int v = 0; v < 32; ++v) {
            if (c0 + v >= a.vectors) break;
            const size_t o = (size_t)(c0 + v) * a.rows + r;
            const float val = __uint_as_float(acc[v]) + bias_v;
            a.out[o] = a.epilogue == ETC_EPILOGUE_RESIDUAL ? a.residual[o] + val : val;
          }
        }
      }
    }
    tc_fence_before();
  } else if (warp == 4 * kGroups) {
    // ------------------------------------------------------------------ activation loader (one lane)
    if (lane == 0) {
      chain_wait();  // the activations come from the kernel before this one; weights do not, the dequant warps run ahead
      int issued = 0;
      for (int i = 0; i < nstages; ++i) {
        const int s = i % kStages;
        const uint32_t round = (uint32_t)(i / kStages);
        if (!mbar_wait(&empty[s], (round & 1) ^ 1, abort_flag)) break;
        const int kb = kb0 + i * kStageBlocks;
        const int valid = min(kStageBlocks, kb1 - kb);
        const uint32_t bytes = (uint32_t)valid * 4u * NV * 16u;  // 4 column groups of 8 per block
        mbar_arrive_expect_tx(&full_b[s], bytes);
        bulk_copy_g2s(b_ring + (size_t)s * kStageBBytes, a.xh + (size_t)kb * 4 * NV * 8, bytes, &full_b[s]);
        issued = i + 1;
      }
      if (*abort_flag) {
        // give up path: let this warp's own bulk copies land (bounded) before shared memory is released
        for (int i = max(0, issued - kStages); i < issued; ++i) {
          const uint32_t parity = (uint32_t)(i / kStages) & 1;
          for (unsigned spin = 0; spin < (1u << 20) && !mbar_try_wait(&full_b[i % kStages], parity); ++spin) __nanosleep(64);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < nstages && ok; ++i) {
        const int s = i % kStages;
        const uint32_t parity = (uint32_t)(i / kStages) & 1;
        ok = mbar_wait(&full_b[s], parity, abort_flag) && mbar_wait(&full_a[s], parity, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const int valid = min(kStageBlocks, kb1 - (kb0 + i * kStageBlocks));
        const uint32_t b_base = smem_u32(b_ring + (size_t)s * kStageBBytes);
        for (int j = 0; j < 2 * valid; ++j) {  // K = 16 per MMA: two column groups of B, 8 TMEM columns of A
          const uint64_t b_desc = make_b_desc(b_base + (uint32_t)j * 2u * NV * 16u, NV * 16u, 128u);
          umma_ts(d_tmem, a_tmem0 + (uint32_t)(s * kAColsPerStage + j * 8), b_desc, kIdesc, (i > 0 || j > 0) ? 1u : 0u);
        }
        tc_commit(&empty[s]);  // arrives when the MMAs above have finished reading this stage
      }
      if (ok) tc_commit(done);
      tc_fence_before();
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(a.status, 0ull, 3ull);  // bounded wait expired
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// f32 [vectors, K] -> xh8 [K/8][NV][8] f16 (rows >= vectors are zero), saturating like the mma.sync path.
// More than NV vectors: chunk c holds vectors c*NV ... in its own [K/8][NV][8] block.
template <int NV>
__global__ void convert_xh8_kernel(const float* __restrict__ x, int vectors, int K, __half* __restrict__ xh) {
  const int per_chunk = (K / 8) * NV;
  const int64_t total = (int64_t)per_chunk * ((vectors + NV - 1) / NV);
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int chunk = (int)(idx / per_chunk), within = (int)(idx - (int64_t)chunk * per_chunk);
    const int kg = within / NV, n = chunk * NV + (within - kg * NV);
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

// Repack raw GGUF rows into the per-thread streaming layout: for row tile t and block kb the 128 rows'
// 16 (Q4_0) or 32 (Q8_0) payload bytes are contiguous, so each warp load instruction is 512 contiguous bytes.
__global__ void repack_umma_kernel(RepackParts parts, int codec, int64_t rows, int64_t rows_padded, int64_t kblocks,
                                   int interleave8, uint32_t* __restrict__ quants, __half* __restrict__ scales) {
  const int64_t total = rows_padded * kblocks;
  const bool kquant = codec >= 11;
  const int bb = codec == 2 ? 18 : (codec == 8 ? 34 : (codec == 11 ? 110 : (codec == 12 ? 144 : (codec == 13 ? 176 : 210))));  // bytes per source block
  const int per_block = kquant ? 8 : 1;                                              // 32-value blocks per source block
  const int words = (codec == 2 || codec == 12) ? 4 : 8;
  const int64_t row_bytes = kblocks / per_block * bb;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / kblocks, kb = idx - r * kblocks;
    const uint8_t* src_row = nullptr;
    if (r < rows) {
      if (interleave8) {
        const int64_t grp = r >> 4, within = r & 15;
        src_row = parts.ptr[within >= 8 ? 1 : 0] + (grp * 8 + (within & 7)) * row_bytes;
      } else {
        int64_t rr = r;
        for (int p = 0; p < parts.n_parts; ++p) {
          if (rr < parts.rows[p]) { src_row = parts.ptr[p] + rr * row_bytes; break; }
          rr -= parts.rows[p];
        }
      }
    }
    const int64_t tile = r / kUmmaRows, row = r % kUmmaRows;
    uint32_t* dst = quants + ((tile * kblocks + kb) * kUmmaRows + row) * words;
    __half scale = __float2half_rn(0.0f), second = __float2half_rn(0.0f);
    if (!src_row) {
      for (int w = 0; w < words; ++w) dst[w] = codec == 2 ? 0x88888888u : 0u;
    } else if (codec == 12) {
      // Q4_K (crates/runtime-cpu/src/quantized.rs:180-199): sub-block `sub` of the 256-value block, value = d*sc*code - dmin*m
      const uint8_t* blk = src_row + (kb >> 3) * bb;
      const int sub = (int)(kb & 7);
      int sc, mn;
      scale_min_k4(sub, blk + 4, sc, mn);
      scale = __float2half_rn(__fmul_rn(fp16_at(blk, 0), (float)sc));
      second = __float2half_rn(__fmul_rn(fp16_at(blk, 2), (float)mn));
      const int pos[8] = {0, 16, 8, 24, 4, 20, 12, 28};
      for (int w = 0; w < 4; ++w) {
        uint32_t word = 0;
        for (int j = 0; j < 8; ++j) {
          const int raw = blk[16 + (sub >> 1) * 32 + 8 * w + j];
          word |= (uint32_t)((sub & 1) ? (raw >> 4) : (raw & 0x0f)) << pos[j];
        }
        dst[w] = word;
      }
    } else if (codec == 11) {
      // Q3_K (quantized.rs:142-176): block `sub` of the 256-value block is groups 2*sub and 2*sub+1 of 16 values,
      // value = d*(scale6 - 32)*(low2 - (high bit clear ? 4 : 0)); stored as int8 codes with one f16 scale per group, the
      // layout of the re-cut Q6_K
      const uint8_t* blk = src_row + (kb >> 3) * bb;
      const int sub = (int)(kb & 7), half = sub >> 2, lane = sub & 3;
      const uint8_t* packed = blk + 96;
      const float d = fp16_at(blk, 108);
      auto group_scale = [&](int g) {
        const int low = g < 8 ? (packed[g] & 0x0f) : (packed[g - 8] >> 4);
        const int high = (packed[8 + g % 4] >> (2 * (g / 4))) & 3;
        return __float2half_rn(__fmul_rn(d, (float)((low | (high << 4)) - 32)));
      };
      scale = group_scale(2 * sub);
      second = group_scale(2 * sub + 1);
      const uint8_t mask = (uint8_t)(1u << (half * 4 + lane));
      for (int w = 0; w < 8; ++w) {
        uint32_t word = 0;
        for (int j = 0; j < 4; ++j) {
          const int v = 4 * w + j;
          const int code = ((blk[32 + half * 32 + v] >> (2 * lane)) & 3) - ((blk[v] & mask) == 0 ? 4 : 0);
          word |= (uint32_t)(code & 0xff) << (8 * j);
        }
        dst[w] = word;
      }
    } else if (codec == 13) {
      // Q5_K (quantized.rs:203-234): sub-block `sub`, value = d*sc*code - dmin*m with a 5-bit code (low nibble + one high
      // bit); stored as int8 codes with (scale, min) per 32 values
      const uint8_t* blk = src_row + (kb >> 3) * bb;
      const int sub = (int)(kb & 7);
      int sc, mn;
      scale_min_k4(sub, blk + 4, sc, mn);
      scale = __float2half_rn(__fmul_rn(fp16_at(blk, 0), (float)sc));
      second = __float2half_rn(__fmul_rn(fp16_at(blk, 2), (float)mn));
      const uint8_t* ql = blk + 48 + (sub >> 1) * 32;
      const uint8_t mask = (uint8_t)(1u << sub);
      for (int w = 0; w < 8; ++w) {
        uint32_t word = 0;
        for (int j = 0; j < 4; ++j) {
          const int v = 4 * w + j;
          const int code = ((sub & 1) ? (ql[v] >> 4) : (ql[v] & 0x0f)) + ((blk[16 + v] & mask) == 0 ? 0 : 16);
          word |= (uint32_t)code << (8 * j);
        }
        dst[w] = word;
      }
    } else if (codec == 14) {
      // Q6_K (quantized.rs:238-261): values 32*sub .. 32*sub+31 of the 256-value block, value = d*scale*(code - 32) with one
      // int8 scale per 16 values
      const uint8_t* blk = src_row + (kb >> 3) * bb;
      const int first = (int)(kb & 7) * 32;
      const int half = first >> 7, quarter = (first & 127) >> 5;
      const uint8_t* ql = blk + half * 64;
      const uint8_t* qh = blk + 128 + half * 32;
      const float d = fp16_at(blk, 208);
      scale = __float2half_rn(__fmul_rn(d, (float)(int)(signed char)blk[192 + half * 8 + quarter * 2]));
      second = __float2half_rn(__fmul_rn(d, (float)(int)(signed char)blk[192 + half * 8 + quarter * 2 + 1]));
      for (int w = 0; w < 8; ++w) {
        uint32_t word = 0;
        for (int j = 0; j < 4; ++j) {
          const int index = 4 * w + j;
          const int low = (quarter & 1) ? ql[index + 32] : ql[index];
          const int low4 = (quarter & 2) ? (low >> 4) : (low & 0x0f);
          const int code = (low4 | (((qh[index] >> (2 * quarter)) & 3) << 4)) - 32;
          word |= (uint32_t)(code & 0xff) << (8 * j);
        }
        dst[w] = word;
      }
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
          dst[w] = word;
        }
      } else {
        for (int w = 0; w < 8; ++w) {
          uint32_t word = 0;
          for (int j = 0; j < 4; ++j) word |= (uint32_t)blk[2 + 4 * w + j] << (8 * j);
          dst[w] = word;
        }
      }
    }
    if (kquant) {
      scales[((tile * kblocks + kb) * kUmmaRows + row) * 2] = scale;
      scales[((tile * kblocks + kb) * kUmmaRows + row) * 2 + 1] = second;
    } else {
      scales[(tile * kblocks + kb) * kUmmaRows + row] = scale;
    }
  }
}

template <int CODEC, int NV>
cudaError_t launch_umma_pass(const UmmaArgs& args, int tiles, int splits, int chunks, cudaStream_t stream) {
  constexpr size_t smem = UmmaCfg<NV>::kSmemBytes;
  auto kernel = qlinear_umma_kernel<CODEC, NV>;
  const cudaError_t attr = opt_in_shared_memory(kernel, smem);
  if (attr != cudaSuccess) return attr;
  // chained: set-up, weight loads and their expansion do not depend on the previous kernel and start under its tail
  return launch_chained(kernel, dim3((unsigned)tiles, (unsigned)splits, (unsigned)chunks), dim3((unsigned)UmmaCfg<NV>::kThreads), smem, stream, args);
}

}  // namespace

cudaError_t launch_repack_umma(const TiledWeight& w, const RepackParts& parts, cudaStream_t stream) {
  const int64_t kblocks = w.columns / 32;
  const int64_t total = w.rows_padded * kblocks;
  if (total == 0) return cudaSuccess;
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 32);
  repack_umma_kernel<<<grid, 256, 0, stream>>>(parts, w.codec, w.rows, w.rows_padded, kblocks, w.interleave8, (uint32_t*)w.quants, w.scales);
  return cudaGetLastError();
}

int umma_vector_pad(int64_t vectors) { return vectors <= 32 ? 32 : (vectors <= 64 ? 64 : (vectors <= 128 ? 128 : 256)); }

UmmaPlan plan_umma(const TiledWeight& w, int64_t vectors, int sm_count) {
  UmmaPlan p;
  p.nv = umma_vector_pad(std::min<int64_t>(vectors, 256));
  p.chunks = (int)std::max<int64_t>(1, (vectors + p.nv - 1) / p.nv);
  p.tiles = (int)(w.rows_padded / kUmmaRows);
  const int kblocks = (int)(w.columns / 32);
  const int kStageBlocks = stage_blocks_for(p.nv);
  const int stages = (kblocks + kStageBlocks - 1) / kStageBlocks;
  const int ctas_per_sm = p.nv <= 64 ? 2 : 1;
  const int target = std::max(1, sm_count) * ctas_per_sm;
  int splits = std::max(1, target / std::max(1, p.tiles * p.chunks));
  splits = std::min(splits, std::max(1, stages / 2));  // at least two stages per split
  const int stages_per_split = (stages + splits - 1) / splits;
  p.blocks_per_split = stages_per_split * kStageBlocks;
  p.splits = (kblocks + p.blocks_per_split - 1) / p.blocks_per_split;
  p.xh_bytes = (size_t)p.chunks * (w.columns / 8) * p.nv * 16;
  p.scratch_bytes = p.splits > 1 ? (size_t)p.chunks * p.splits * p.nv * w.rows_padded * sizeof(float) : 0;
  return p;
}

// qlinear_reduce_kernel lives in quant_kernels.cu
cudaError_t launch_qlinear_umma(const TiledWeight& w, const float* x, const __half* xh_ready, int64_t vectors, const float* bias,
                                const float* residual, int epilogue, float* out, __half* out_xh, __half* xh, float* scratch,
                                DeviceStatus* status, int sm_count, cudaStream_t stream, int* launches, int xh_nv, DeferredSum* defer) {
  if (defer) *defer = DeferredSum();
  if (vectors <= 0) return cudaSuccess;
  const int out_cols = (int)(epilogue == ETC_EPILOGUE_SWIGLU ? w.rows / 2 : w.rows);
  const UmmaPlan plan = plan_umma(w, vectors, sm_count);
  const int K = (int)w.columns;
  const int64_t total = (int64_t)(K / 8) * plan.nv * plan.chunks;
  const unsigned cgrid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8);
  const bool ready = xh_ready != nullptr && vectors <= 128 && plan.nv == xh_nv;  // the producer stored the f16 layout with this row stride
  if (!ready) switch (plan.nv) {
    case 32: convert_xh8_kernel<32><<<cgrid, 256, 0, stream>>>(x, (int)vectors, K, xh); break;
    case 64: convert_xh8_kernel<64><<<cgrid, 256, 0, stream>>>(x, (int)vectors, K, xh); break;
    case 128: convert_xh8_kernel<128><<<cgrid, 256, 0, stream>>>(x, (int)vectors, K, xh); break;
    default: convert_xh8_kernel<256><<<cgrid, 256, 0, stream>>>(x, (int)vectors, K, xh); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (launches && !ready) ++*launches;
  UmmaArgs args;
  args.quants = reinterpret_cast<const uint4*>(w.quants);
  args.scales = w.scales;
  args.xh = ready ? xh_ready : xh;
  args.out_xh = vectors <= xh_nv ? out_xh : nullptr;
  args.out_xh_nv = xh_nv;
  args.bias = bias;
  args.residual = residual;
  args.out = out;
  args.scratch = scratch;
  args.status = &status->code;
  args.vectors = (int)vectors;
  args.rows = (int)w.rows;
  args.rows_padded = (int)w.rows_padded;
  args.kblocks = K / 32;
  args.blocks_per_split = plan.blocks_per_split;
  args.epilogue = epilogue;
  args.tile0 = 0;
  int codec = w.codec, tiles = plan.tiles;
  auto pass = [&](auto nv_tag) {
    constexpr int NV = decltype(nv_tag)::value;
    switch (codec) {
      case 2: return launch_umma_pass<2, NV>(args, tiles, plan.splits, plan.chunks, stream);
      case 8: return launch_umma_pass<8, NV>(args, tiles, plan.splits, plan.chunks, stream);
      case 12: return launch_umma_pass<12, NV>(args, tiles, plan.splits, plan.chunks, stream);
      case 13: return launch_umma_pass<13, NV>(args, tiles, plan.splits, plan.chunks, stream);
      default:  // 14, and 11 whose re-cut form is the same
        return launch_umma_pass<14, NV>(args, tiles, plan.splits, plan.chunks, stream);
    }
  };
  // one launch per run of equal codecs; all of them share the plan (split count, partial layout) of the whole weight
  const int n_segments = std::max(1, w.n_segments);
  for (int sgm = 0; sgm < n_segments; ++sgm) {
    if (w.n_segments > 0) {
      const TiledSegment& seg = w.segments[sgm];
      codec = seg.codec;
      tiles = seg.tiles;
      args.tile0 = seg.tile0;
      args.quants = reinterpret_cast<const uint4*>(w.quants + seg.quant_offset);
      args.scales = reinterpret_cast<const __half*>(reinterpret_cast<const uint8_t*>(w.scales) + seg.scale_offset);
    }
    switch (plan.nv) {
      case 32: e = pass(std::integral_constant<int, 32>()); break;
      case 64: e = pass(std::integral_constant<int, 64>()); break;
      case 128: e = pass(std::integral_constant<int, 128>()); break;
      default: e = pass(std::integral_constant<int, 256>()); break;
    }
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  if (plan.splits > 1 && defer && plan.chunks == 1 && !bias && !out_xh && epilogue != ETC_EPILOGUE_SWIGLU) {
    // the consumer sums the partials itself (and adds the residual stream where the epilogue asks for it)
    defer->partials = scratch;
    defer->splits = plan.splits;
    defer->vpad = plan.nv;
    defer->rows_padded = (int)w.rows_padded;
  } else if (plan.splits > 1) {
    for (int c = 0; c < plan.chunks; ++c) {  // one sum launch per chunk of vectors
      const int64_t v0 = (int64_t)c * plan.nv;
      const float* partials = scratch + (size_t)c * plan.splits * plan.nv * w.rows_padded;
      e = launch_qlinear_reduce(partials, plan.splits, plan.nv, (int)std::min<int64_t>(plan.nv, vectors - v0), (int)w.rows, (int)w.rows_padded,
                                bias, residual ? residual + v0 * out_cols : nullptr, epilogue, out + v0 * out_cols, c == 0 ? args.out_xh : nullptr,
                                stream, xh_nv);
      if (e != cudaSuccess) return e;
      if (launches) ++*launches;
    }
  }
  return cudaSuccess;
}

}  // namespace etc
