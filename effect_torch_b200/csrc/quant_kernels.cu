// Block-quantized weight kernels for sm_100a: dequantise, quantise, the generic (any codec, raw
// GGUF layout) linear, the row-gather embedding, the repack into the tensor-core tiling and the
// tiled dequant-matvec/GEMM that the decode step runs on.
//
// Replaces crates/runtime-cpu/src/quantized.rs (decode_block :90, linear_into :419,
// embedding_into :546) of the reference for the CUDA backend.
#include <cuda_fp16.h>
#include <mma.h>

#include <algorithm>

#include "codecs.cuh"
#include "chain.cuh"
#include "kernels.h"

namespace etc {

// ============================================================================================
// Dequantise / embedding: one thread per output element, bit-exact with the reference decoders.
// HBM-bound on the f32 output (4 B written per 0.5-1 B read).
// ============================================================================================
template <int CODEC>
__global__ void dequantize_kernel(const uint8_t* __restrict__ packed, int64_t rows, int64_t columns,
                                  float* __restrict__ out) {
  constexpr int BV = CodecTraits<CODEC>::kValues, BB = CodecTraits<CODEC>::kBytes;
  const int64_t blocks_per_row = columns / BV;
  const int64_t total = rows * columns;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / columns, col = idx - row * columns;
    const uint8_t* block = packed + (row * blocks_per_row + col / BV) * BB;
    out[idx] = decode_elem<CODEC>(block, (int)(col % BV));
  }
}

struct DequantLaunch {
  const uint8_t* packed; int64_t rows, columns; float* out; cudaStream_t stream; cudaError_t err;
  template <int CODEC> void operator()() {
    const int64_t total = rows * columns;
    const int threads = 256;
    const int64_t blocks = std::min<int64_t>((total + threads - 1) / threads, 148 * 32);
    if (total == 0) { err = cudaSuccess; return; }
    dequantize_kernel<CODEC><<<(unsigned)blocks, threads, 0, stream>>>(packed, rows, columns, out);
    err = cudaGetLastError();
  }
};
cudaError_t launch_dequantize(int codec, const uint8_t* packed, int64_t rows, int64_t columns, float* out,
                              cudaStream_t stream) {
  DequantLaunch l{packed, rows, columns, out, stream, cudaSuccess};
  if (!dispatch_codec(codec, l)) return cudaErrorInvalidValue;
  return l.err;
}

template <int CODEC, typename Index>
__global__ void qembedding_kernel(const Index* __restrict__ indexes, int64_t count, const uint8_t* __restrict__ packed,
                                  int64_t rows, int64_t columns, float* __restrict__ out, DeviceStatus* status) {
  constexpr int BV = CodecTraits<CODEC>::kValues, BB = CodecTraits<CODEC>::kBytes;
  const int64_t blocks_per_row = columns / BV;
  const int64_t i = blockIdx.y;
  if (i >= count) return;
  const long long row = (long long)indexes[i];
  if (row < 0 || row >= rows) {  // recorded, never trapped: the host reports it after the stream sync
    if (threadIdx.x == 0 && blockIdx.x == 0 && atomicCAS(&status->code, kStatusNone, kStatusIndexOutOfRange) == kStatusNone) {
      status->value = row;
      status->bound = rows;
    }
    return;
  }
  for (int64_t col = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; col < columns; col += (int64_t)gridDim.x * blockDim.x) {
    const uint8_t* block = packed + (row * blocks_per_row + col / BV) * BB;
    out[i * columns + col] = decode_elem<CODEC>(block, (int)(col % BV));
  }
}

struct EmbeddingLaunch {
  const void* indexes; int is_i64; int64_t count; const uint8_t* weight; int64_t rows, columns; float* out;
  DeviceStatus* status; cudaStream_t stream; cudaError_t err;
  template <int CODEC> void operator()() {
    if (count == 0) { err = cudaSuccess; return; }
    const int threads = 256;
    dim3 grid((unsigned)std::min<int64_t>((columns + threads - 1) / threads, 64), (unsigned)count);
    if (is_i64)
      qembedding_kernel<CODEC, long long><<<grid, threads, 0, stream>>>((const long long*)indexes, count, weight, rows, columns, out, status);
    else
      qembedding_kernel<CODEC, unsigned int><<<grid, threads, 0, stream>>>((const unsigned int*)indexes, count, weight, rows, columns, out, status);
    err = cudaGetLastError();
  }
};
cudaError_t launch_qembedding(int codec, const void* indexes, int index_is_i64, int64_t count, const uint8_t* weight,
                              int64_t rows, int64_t columns, float* out, DeviceStatus* status, cudaStream_t stream) {
  EmbeddingLaunch l{indexes, index_is_i64, count, weight, rows, columns, out, status, stream, cudaSuccess};
  if (!dispatch_codec(codec, l)) return cudaErrorInvalidValue;
  return l.err;
}

// ============================================================================================
// Quantisers (the reference has none). One warp per 32-value block.
//   Q4_0: the element of largest magnitude, signed, divided by -8 is the scale d (so the extreme
//         maps to code 0); stored as f16; code = clamp(floor(x * (1/d) + 8.5), 0, 15) using the
//         unrounded f32 d; ties between equal magnitudes keep the first element.
//   Q8_0: d = absmax / 127 stored as f16; code = clamp(round-half-away(x * (1/d)), -127, 127).
// ============================================================================================
__global__ void quantize_q4_0_kernel(const float* __restrict__ x, int64_t total_blocks, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t blk = warp; blk < total_blocks; blk += nwarps) {
    const float v = x[blk * 32 + lane];
    float amax = fabsf(v);
    int arg = lane;
    // max magnitude, first index on ties
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
      const int oi = __shfl_xor_sync(0xffffffffu, arg, off);
      if (oa > amax || (oa == amax && oi < arg)) { amax = oa; arg = oi; }
    }
    const float extreme = amax > 0.0f ? __shfl_sync(0xffffffffu, v, arg) : 0.0f;
    const float d = __fdiv_rn(extreme, -8.0f);
    const float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int code = (int)floorf(__fadd_rn(__fmul_rn(v, inv), 8.5f));
    code = code < 0 ? 0 : (code > 15 ? 15 : code);
    const int hi = __shfl_down_sync(0xffffffffu, code, 16);
    uint8_t* dst = out + blk * 18;
    if (lane < 16) dst[2 + lane] = (uint8_t)(code | (hi << 4));
    if (lane == 0) {
      // block offsets are even, so the little-endian f16 scale is one aligned 16-bit store
      *reinterpret_cast<unsigned short*>(dst) = __half_as_ushort(__float2half_rn(d));
    }
  }
}

__global__ void quantize_q8_0_kernel(const float* __restrict__ x, int64_t total_blocks, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t blk = warp; blk < total_blocks; blk += nwarps) {
    const float v = x[blk * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float d = __fdiv_rn(amax, 127.0f);
    const float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    float q = roundf(__fmul_rn(v, inv));
    q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
    uint8_t* dst = out + blk * 34;
    dst[2 + lane] = (uint8_t)(signed char)(int)q;
    if (lane == 0) {
      // block offsets are even, so the little-endian f16 scale is one aligned 16-bit store
      *reinterpret_cast<unsigned short*>(dst) = __half_as_ushort(__float2half_rn(d));
    }
  }
}

cudaError_t launch_quantize(int codec, const float* x, int64_t rows, int64_t columns, uint8_t* packed,
                            cudaStream_t stream) {
  const int64_t blocks = rows * (columns / 32);
  if (blocks == 0) return cudaSuccess;
  const int threads = 256;
  const unsigned grid = (unsigned)std::min<int64_t>((blocks + 7) / 8, 148 * 16);
  if (codec == kQ4_0) quantize_q4_0_kernel<<<grid, threads, 0, stream>>>(x, blocks, packed);
  else if (codec == kQ8_0) quantize_q8_0_kernel<<<grid, threads, 0, stream>>>(x, blocks, packed);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ============================================================================================
// Generic linear on the raw GGUF layout (every codec). One warp per weight row; the warp walks
// the row 256 values at a time, lane l decoding elements l, l+32, ... of the window so the
// activation reads are coalesced; up to VC input vectors are accumulated per pass so the packed
// row is read once per VC vectors. f32 accumulation, shuffle reduction. HBM-bound for small
// vector counts; not the decode-step path (that is the tiled kernel below).
// ============================================================================================
template <int CODEC, int VC>
__global__ void __launch_bounds__(256) qlinear_generic_kernel(const float* __restrict__ x, int vectors, int64_t columns,
                                                              const uint8_t* __restrict__ weight, int64_t rows,
                                                              const float* __restrict__ bias, float* __restrict__ out) {
  constexpr int BV = CodecTraits<CODEC>::kValues, BB = CodecTraits<CODEC>::kBytes;
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t row_bytes = columns / BV * BB;
  const uint8_t* wrow = weight + row * row_bytes;
  float acc[VC];
#pragma unroll
  for (int v = 0; v < VC; ++v) acc[v] = 0.0f;
  for (int64_t base = 0; base < columns; base += 256) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t col = base + lane + 32 * j;
      if (col < columns) {
        const float w = decode_elem<CODEC>(wrow + (col / BV) * BB, (int)(col % BV));
#pragma unroll
        for (int v = 0; v < VC; ++v)
          if (v < vectors) acc[v] = fmaf(x[(int64_t)v * columns + col], w, acc[v]);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VC; ++v) {
    float s = acc[v];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0 && v < vectors) out[(int64_t)v * rows + row] = s + (bias ? bias[row] : 0.0f);
  }
}

struct GenericLaunch {
  const float* x; int64_t vectors, columns; const uint8_t* weight; int64_t rows; const float* bias; float* out;
  cudaStream_t stream; cudaError_t err; int launches;
  template <int CODEC> void operator()() {
    constexpr int VC = 8;
    err = cudaSuccess;
    if (rows == 0) return;
    const unsigned grid = (unsigned)((rows + 7) / 8);
    for (int64_t v0 = 0; v0 < vectors; v0 += VC) {
      const int chunk = (int)std::min<int64_t>(VC, vectors - v0);
      qlinear_generic_kernel<CODEC, VC><<<grid, 256, 0, stream>>>(x + v0 * columns, chunk, columns, weight, rows, bias,
                                                                    out + v0 * rows);
      ++launches;
      err = cudaGetLastError();
      if (err != cudaSuccess) return;
    }
  }
};
cudaError_t launch_qlinear_generic(int codec, const float* x, int64_t vectors, int64_t columns, const uint8_t* weight,
                                   int64_t rows, const float* bias, float* out, cudaStream_t stream, int* launches) {
  GenericLaunch l{x, vectors, columns, weight, rows, bias, out, stream, cudaSuccess, 0};
  if (!dispatch_codec(codec, l)) return cudaErrorInvalidValue;
  if (launches) *launches += l.launches;
  return l.err;
}

// ============================================================================================
// Tensor-core tiling of Q4_0 / Q8_0 weights.
//
// Rows are grouped in tiles of 16 (one mma.m16n8k16 A operand height), columns in 32-value
// blocks (kb). Inside the kernel, lane (g = lane/4, t = lane%4) of a warp owns rows g and g+8 of
// a tile and logical columns kb*32 + 8t .. 8t+7 of each block: four of them feed the first
// k16 MMA of the block and four the second, in the same order the activation fragment is read
// from shared memory (columns 8t..8t+3 then 8t+4..8t+7), so activations stay in natural order.
//
//   Q4_0 quants: [row_tile][kb/2][lane][16 B] = {kb0 row g, kb0 row g+8, kb1 row g, kb1 row g+8},
//                each u32 holding the lane's 8 nibbles with logical column j of the lane at bit
//                position {0,16,8,24,4,20,12,28}[j] (so masking with 0x000F000F / 0x00F000F0 after
//                shifting by 0 or 8 yields ready-made half2 operand pairs).
//        scales: [row_tile][kb/2][g][4] f16 = {kb0 row g, kb0 row g+8, kb1 row g, kb1 row g+8}.
//   Q8_0 quants: [row_tile][kb][lane][16 B] = {row g cols 8t..8t+3, row g cols 8t+4..8t+7,
//                row g+8 cols 8t..8t+3, row g+8 cols 8t+4..8t+7} as int8.
//        scales: [row_tile][kb][g][2] f16 = {row g, row g+8}.
// Byte count equals the GGUF encoding (18 resp. 34 bytes per block); rows are padded to 16 with
// zero scales. A warp's loads are 512 contiguous bytes.
// ============================================================================================
__device__ __forceinline__ const uint8_t* part_row(const RepackParts& parts, int64_t r, int64_t total_rows,
                                                   int interleave8, int64_t row_bytes) {
  if (r >= total_rows) return nullptr;
  if (interleave8) {
    const int64_t grp = r >> 4, within = r & 15;
    const int part = within >= 8 ? 1 : 0;
    return parts.ptr[part] + (grp * 8 + (within & 7)) * row_bytes;
  }
  int64_t rr = r;
  for (int p = 0; p < parts.n_parts; ++p) {
    if (rr < parts.rows[p]) return parts.ptr[p] + rr * row_bytes;
    rr -= parts.rows[p];
  }
  return nullptr;
}

__global__ void repack_q4_0_kernel(RepackParts parts, int64_t rows, int64_t rows_padded, int64_t kblocks, int interleave8,
                                   uint32_t* __restrict__ quants, __half* __restrict__ scales) {
  const int64_t total = rows_padded * kblocks;
  const int64_t kbp_count = kblocks / 2;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / kblocks, kb = idx - r * kblocks;
    const uint8_t* src_row = part_row(parts, r, rows, interleave8, kblocks * 18);
    const int64_t rt = r >> 4;
    const int rr = (int)(r & 15), g = rr & 7, hi8 = rr >> 3;
    const int64_t kbp = kb >> 1;
    const int h = (int)(kb & 1);
    uint32_t words[4] = {0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};
    __half scale = __float2half_rn(0.0f);
    if (src_row) {
      const uint8_t* blk = src_row + kb * 18;
      scale = __ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8)));
      const int pos[8] = {0, 16, 8, 24, 4, 20, 12, 28};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = 8 * t + j;  // logical element of the block
          const uint32_t code = i < 16 ? (blk[2 + i] & 0x0fu) : (uint32_t)(blk[2 + i - 16] >> 4);
          w |= code << pos[j];
        }
        words[t] = w;
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int lane = g * 4 + t;
      quants[((rt * kbp_count + kbp) * 32 + lane) * 4 + (h * 2 + hi8)] = words[t];
    }
    scales[((rt * kbp_count + kbp) * 8 + g) * 4 + (h * 2 + hi8)] = scale;
  }
}

__global__ void repack_q8_0_kernel(RepackParts parts, int64_t rows, int64_t rows_padded, int64_t kblocks, int interleave8,
                                   uint32_t* __restrict__ quants, __half* __restrict__ scales) {
  const int64_t total = rows_padded * kblocks;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / kblocks, kb = idx - r * kblocks;
    const uint8_t* src_row = part_row(parts, r, rows, interleave8, kblocks * 34);
    const int64_t rt = r >> 4;
    const int rr = (int)(r & 15), g = rr & 7, hi8 = rr >> 3;
    __half scale = __float2half_rn(0.0f);
    const uint8_t* blk = nullptr;
    if (src_row) {
      blk = src_row + kb * 34;
      scale = __ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8)));
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t w0 = 0, w1 = 0;
      if (blk) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          w0 |= (uint32_t)blk[2 + 8 * t + j] << (8 * j);
          w1 |= (uint32_t)blk[2 + 8 * t + 4 + j] << (8 * j);
        }
      }
      const int lane = g * 4 + t;
      uint32_t* dst = quants + ((rt * kblocks + kb) * 32 + lane) * 4 + hi8 * 2;
      dst[0] = w0;
      dst[1] = w1;
    }
    scales[((rt * kblocks + kb) * 8 + g) * 2 + hi8] = scale;
  }
}

cudaError_t launch_repack(const TiledWeight& w, const RepackParts& parts, cudaStream_t stream) {
  if (w.layout == kLayoutUmma128) return launch_repack_umma(w, parts, stream);
  if (w.layout == kLayoutStream256) return launch_repack_stream(w, parts, stream);
  const int64_t kblocks = w.columns / 32;
  const int64_t total = w.rows_padded * kblocks;
  if (total == 0) return cudaSuccess;
  const int threads = 256;
  const unsigned grid = (unsigned)std::min<int64_t>((total + threads - 1) / threads, 148 * 32);
  if (w.codec == kQ4_0)
    repack_q4_0_kernel<<<grid, threads, 0, stream>>>(parts, w.rows, w.rows_padded, kblocks, w.interleave8, (uint32_t*)w.quants, w.scales);
  else if (w.codec == kQ8_0)
    repack_q8_0_kernel<<<grid, threads, 0, stream>>>(parts, w.rows, w.rows_padded, kblocks, w.interleave8, (uint32_t*)w.quants, w.scales);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ============================================================================================
// Tiled dequant linear on tensor cores (mma.sync m16n8k16, f16 operands, f32 accumulate).
//
// out[v, r] = sum_k x[v,k] * W[r,k]. The weight is the A operand (16 rows per tile), the input
// vectors are the B operand (8 per n-tile, NT n-tiles = up to 32 vectors per pass), so no MMA row
// is wasted on padding for decode batches. A CTA is 8 warps; warp w owns MT row tiles and walks
// the CTA's K range; activations for the range are staged once per CTA into shared memory as f16
// (chunks of KC columns) and read back as B fragments with one 16-byte load per (n-tile, block).
// Packed weights stream global -> registers with 16-byte coalesced loads (prefetched PF block
// groups ahead) and are expanded to f16 in registers: nibbles are spliced into the mantissa of
// 1024.0h (lop3) and rebased with one hsub2/hfma2, then scaled by the block scale (hmul2).
// Split-K (grid.y) spreads small matrices over all SMs: partial sums go to a scratch buffer and a
// second kernel reduces them and applies the epilogue; with one split the epilogue runs in place.
//
// Roofline: HBM-bound up to 32 vectors: algorithmic bytes = rows*(K/32)*{18,34} + 4*V*K + 4*V*rows.
// ============================================================================================
constexpr int kTiledWarps = 8;
constexpr int kTiledKC = 1024;                  // activation columns staged per chunk
constexpr int kTiledXStride = kTiledKC + 32;    // halves; row stride = 2112 B = 64 (mod 128): conflict-free 16 B reads

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// One packed u32 of a Q4_0 lane (8 nibbles, see layout above) -> four half2: {c0,c1},{c2,c3} for the
// block's first MMA and {c4,c5},{c6,c7} for the second, already multiplied by the block scale.
__device__ __forceinline__ void dequant_q4_word(uint32_t q, __half2 scale, uint32_t& lo0, uint32_t& lo1, uint32_t& hi0,
                                                uint32_t& hi1) {
  const uint32_t kMagic = 0x64006400u;  // half2(1024, 1024)
  const uint32_t qs = q >> 8;
  const __half2 bias_lo = __floats2half2_rn(1032.0f, 1032.0f);       // 1024 + 8
  const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 bias_hi = __floats2half2_rn(-72.0f, -72.0f);          // -(1024/16 + 8)
  const __half2 a = __hsub2(u32_as_h2((q & 0x000F000Fu) | kMagic), bias_lo);
  const __half2 b = __hsub2(u32_as_h2((qs & 0x000F000Fu) | kMagic), bias_lo);
  const __half2 c = __hfma2(u32_as_h2((q & 0x00F000F0u) | kMagic), sixteenth, bias_hi);
  const __half2 d = __hfma2(u32_as_h2((qs & 0x00F000F0u) | kMagic), sixteenth, bias_hi);
  lo0 = h2_as_u32(__hmul2(a, scale));
  lo1 = h2_as_u32(__hmul2(b, scale));
  hi0 = h2_as_u32(__hmul2(c, scale));
  hi1 = h2_as_u32(__hmul2(d, scale));
}

// Four int8 -> two half2 {b0,b1},{b2,b3} times scale: bytes are biased to unsigned (xor 0x80),
// spliced under the exponent byte 0x64 (prmt) giving 1024 + (b + 128), then rebased exactly.
__device__ __forceinline__ void dequant_q8_word(uint32_t w, __half2 scale, uint32_t& p0, uint32_t& p1) {
  const uint32_t x = w ^ 0x80808080u;
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
  const __half2 a = __hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4140)), bias);
  const __half2 b = __hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4342)), bias);
  p0 = h2_as_u32(__hmul2(a, scale));
  p1 = h2_as_u32(__hmul2(b, scale));
}

__device__ __forceinline__ float silu_tanh_form(float x) { return x * (tanhf(x * 0.5f) * 0.5f + 0.5f); }

struct TiledArgs {
  const uint8_t* quants;
  const __half* scales;
  const float* x;         // [vectors, K] f32
  const float* bias;      // logical rows (pre-epilogue), may be null
  const float* residual;  // [vectors, out_cols] when epilogue == RESIDUAL
  float* out;             // [vectors, out_cols]
  float* scratch;         // [splits][NT*8][rows_padded]
  int vectors;
  int rows;               // logical rows
  int rows_padded;
  int K;
  int row_tiles;
  int units;              // number of weight load units along K (kb pairs for Q4_0, kb for Q8_0)
  int units_per_split;
  int epilogue;
};

template <int CODEC, int MT, int NT>
__global__ void __launch_bounds__(kTiledWarps * 32, 2) qlinear_tiled_kernel(TiledArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);  // [NT*8][kTiledXStride]
  constexpr int KB_PER_UNIT = CODEC == kQ4_0 ? 2 : 1;   // 32-column blocks per 16-byte lane load
  constexpr int PF = 2;                                   // load units prefetched ahead
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int unit0 = blockIdx.y * a.units_per_split;
  const int unit1 = min(a.units, unit0 + a.units_per_split);
  const int rt0 = (blockIdx.x * kTiledWarps + warp) * MT;

  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.0f;

  // per-row-tile base pointers (tiles past the end are clamped for loads and masked at the store)
  const uint4* qbase[MT];
  const uint8_t* sbase[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int rt = min(rt0 + mt, a.row_tiles - 1);
    qbase[mt] = reinterpret_cast<const uint4*>(a.quants) + (size_t)rt * a.units * 32 + lane;
    sbase[mt] = reinterpret_cast<const uint8_t*>(a.scales) + ((size_t)rt * a.units * 8 + g) * (KB_PER_UNIT * 4);
  }
  const bool warp_active = rt0 < a.row_tiles;

  constexpr int UNITS_PER_CHUNK = kTiledKC / (32 * KB_PER_UNIT);
  for (int cu0 = unit0; cu0 < unit1; cu0 += UNITS_PER_CHUNK) {
    const int cu1 = min(unit1, cu0 + UNITS_PER_CHUNK);
    const int k_begin = cu0 * 32 * KB_PER_UNIT;
    const int k_len = (cu1 - cu0) * 32 * KB_PER_UNIT;
    __syncthreads();  // previous chunk fully consumed
    // ---- stage activations: f32 -> f16 (saturating), rows >= vectors are zero
    for (int idx = threadIdx.x * 4; idx < NT * 8 * k_len; idx += kTiledWarps * 32 * 4) {
      const int v = idx / k_len, kk = idx - v * k_len;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (v < a.vectors) val = *reinterpret_cast<const float4*>(a.x + (size_t)v * a.K + k_begin + kk);
      __half2 h01 = __floats2half2_rn(fminf(fmaxf(val.x, -65504.f), 65504.f), fminf(fmaxf(val.y, -65504.f), 65504.f));
      __half2 h23 = __floats2half2_rn(fminf(fmaxf(val.z, -65504.f), 65504.f), fminf(fmaxf(val.w, -65504.f), 65504.f));
      uint2 packed = make_uint2(h2_as_u32(h01), h2_as_u32(h23));
      *reinterpret_cast<uint2*>(xs + (size_t)v * kTiledXStride + kk) = packed;
    }
    __syncthreads();
    if (!warp_active) continue;

    // ---- stream weight units cu0..cu1 with a PF-deep register prefetch
    uint4 qbuf[PF][MT];
    uint2 sbuf[PF][MT];
#pragma unroll
    for (int s = 0; s < PF; ++s) {
      const int u = min(cu0 + s, cu1 - 1);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        qbuf[s][mt] = __ldg(qbase[mt] + (size_t)u * 32);
        if (CODEC == kQ4_0) sbuf[s][mt] = __ldg(reinterpret_cast<const uint2*>(sbase[mt] + (size_t)u * 64));
        else sbuf[s][mt].x = __ldg(reinterpret_cast<const uint32_t*>(sbase[mt] + (size_t)u * 32));
      }
    }
    for (int ub = cu0; ub < cu1; ub += PF) {
#pragma unroll
      for (int s = 0; s < PF; ++s) {
        const int u = ub + s;
        if (u < cu1) {
          uint4 qv[MT];
          uint2 sv[MT];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) { qv[mt] = qbuf[s][mt]; sv[mt] = sbuf[s][mt]; }
          // refill this slot for unit u + PF
          {
            const int un = min(u + PF, cu1 - 1);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              qbuf[s][mt] = __ldg(qbase[mt] + (size_t)un * 32);
              if (CODEC == kQ4_0) sbuf[s][mt] = __ldg(reinterpret_cast<const uint2*>(sbase[mt] + (size_t)un * 64));
              else sbuf[s][mt].x = __ldg(reinterpret_cast<const uint32_t*>(sbase[mt] + (size_t)un * 32));
            }
          }
#pragma unroll
          for (int h = 0; h < KB_PER_UNIT; ++h) {
            const int kloc = ((u - cu0) * KB_PER_UNIT + h) * 32 + 8 * t;  // column inside the staged chunk
            uint32_t a_lo[MT][4], a_hi[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              if (CODEC == kQ4_0) {
                const uint32_t wg = h == 0 ? qv[mt].x : qv[mt].z;
                const uint32_t wg8 = h == 0 ? qv[mt].y : qv[mt].w;
                const __half2 sc = u32_as_h2(h == 0 ? sv[mt].x : sv[mt].y);  // {row g, row g+8}
                const __half2 sg = __low2half2(sc), sg8 = __high2half2(sc);
                dequant_q4_word(wg, sg, a_lo[mt][0], a_lo[mt][2], a_hi[mt][0], a_hi[mt][2]);
                dequant_q4_word(wg8, sg8, a_lo[mt][1], a_lo[mt][3], a_hi[mt][1], a_hi[mt][3]);
              } else {
                const __half2 sc = u32_as_h2(sv[mt].x);
                const __half2 sg = __low2half2(sc), sg8 = __high2half2(sc);
                dequant_q8_word(qv[mt].x, sg, a_lo[mt][0], a_lo[mt][2]);
                dequant_q8_word(qv[mt].y, sg, a_hi[mt][0], a_hi[mt][2]);
                dequant_q8_word(qv[mt].z, sg8, a_lo[mt][1], a_lo[mt][3]);
                dequant_q8_word(qv[mt].w, sg8, a_hi[mt][1], a_hi[mt][3]);
              }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint4 bv = *reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + g) * kTiledXStride + kloc);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                mma_f16(acc[mt][nt], a_lo[mt], bv.x, bv.y);
                mma_f16(acc[mt][nt], a_hi[mt], bv.z, bv.w);
              }
            }
          }
        }
      }
    }
  }

  if (!warp_active) return;
  // ---- epilogue. acc[mt][nt] = {(row g, vec 2t), (row g, vec 2t+1), (row g+8, vec 2t), (row g+8, vec 2t+1)}
  const bool direct = gridDim.y == 1;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int rt = rt0 + mt;
    if (rt >= a.row_tiles) continue;
    const int r_lo = rt * 16 + g, r_hi = r_lo + 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int v = nt * 8 + 2 * t + j;
        float lo = acc[mt][nt][j], hi = acc[mt][nt][2 + j];
        if (!direct) {
          float* dst = a.scratch + ((size_t)blockIdx.y * (NT * 8) + v) * a.rows_padded;
          dst[r_lo] = lo;
          dst[r_hi] = hi;
          continue;
        }
        if (v >= a.vectors) continue;
        if (a.bias) {
          if (r_lo < a.rows) lo += a.bias[r_lo];
          if (r_hi < a.rows) hi += a.bias[r_hi];
        }
        if (a.epilogue == ETC_EPILOGUE_SWIGLU) {
          const int oc = rt * 8 + g;  // gate row r_lo pairs with up row r_hi
          if (r_hi < a.rows) a.out[(size_t)v * (a.rows / 2) + oc] = silu_tanh_form(lo) * hi;
        } else {
          if (r_lo < a.rows) {
            const size_t o = (size_t)v * a.rows + r_lo;
            a.out[o] = a.epilogue == ETC_EPILOGUE_RESIDUAL ? a.residual[o] + lo : lo;
          }
          if (r_hi < a.rows) {
            const size_t o = (size_t)v * a.rows + r_hi;
            a.out[o] = a.epilogue == ETC_EPILOGUE_RESIDUAL ? a.residual[o] + hi : hi;
          }
        }
      }
    }
  }
}

// Sums the split-K partials in split order (deterministic) and applies bias / epilogue.
// `residual` and `out` may be the same buffer (the decoder adds projections onto its hidden state in place), so
// neither carries a no-alias promise.
__global__ void qlinear_reduce_kernel(const float* __restrict__ scratch, int splits, int vpad, int vectors, int rows,
                                      int rows_padded, const float* __restrict__ bias, const float* residual,
                                      int epilogue, float* out, __half* __restrict__ out_xh, int xh_nv) {
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  chain_wait();
  const int out_cols = epilogue == ETC_EPILOGUE_SWIGLU ? rows / 2 : rows;
  const int64_t total = (int64_t)vectors * out_cols;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx / out_cols), c = (int)(idx - (int64_t)v * out_cols);
    if (epilogue == ETC_EPILOGUE_SWIGLU) {
      const int r_gate = (c >> 3) * 16 + (c & 7), r_up = r_gate + 8;
      float gsum = 0.f, usum = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float* p = scratch + ((size_t)s * vpad + v) * rows_padded;
        gsum += p[r_gate];
        usum += p[r_up];
      }
      if (bias) { gsum += bias[r_gate]; usum += bias[r_up]; }
      const float act = silu_tanh_form(gsum) * usum;
      if (out) out[idx] = act;
      if (out_xh)  // f16 copy in [cols/8][xh_nv][8] order: the next linear's B operand
        out_xh[((size_t)(c >> 3) * xh_nv + v) * 8 + (c & 7)] = __float2half_rn(fminf(fmaxf(act, -65504.f), 65504.f));
    } else {
      float sum = 0.f;
      for (int s = 0; s < splits; ++s) sum += scratch[((size_t)s * vpad + v) * rows_padded + c];
      if (bias) sum += bias[c];
      const float val = epilogue == ETC_EPILOGUE_RESIDUAL ? residual[idx] + sum : sum;
      if (out) out[idx] = val;
      if (out_xh) out_xh[((size_t)(c >> 3) * xh_nv + v) * 8 + (c & 7)] = __float2half_rn(fminf(fmaxf(val, -65504.f), 65504.f));
    }
  }
}

TiledPlan plan_tiled(const TiledWeight& w, int64_t vectors, int sm_count) {
  TiledPlan p;
  const int64_t v = std::min<int64_t>(vectors, 32);
  p.nt = v <= 8 ? 1 : (v <= 16 ? 2 : 4);
  constexpr int MT = 2;
  const int row_tiles = (int)(w.rows_padded / 16);
  p.grid_x = (row_tiles + kTiledWarps * MT - 1) / (kTiledWarps * MT);
  const int units = (int)(w.columns / (w.codec == kQ4_0 ? 64 : 32));
  const int min_units = w.codec == kQ4_0 ? 4 : 8;  // at least 256 columns per split
  const int target = std::max(1, sm_count) * 2;
  int splits = std::max(1, target / p.grid_x);
  splits = std::min(splits, std::max(1, units / min_units));
  const int ups = (units + splits - 1) / splits;
  p.splits = (units + ups - 1) / ups;
  p.scratch_bytes = p.splits > 1 ? (size_t)p.splits * (p.nt * 8) * w.rows_padded * sizeof(float) : 0;
  return p;
}

template <int CODEC, int NT>
static cudaError_t launch_tiled_pass(const TiledWeight& w, const TiledPlan& plan, TiledArgs args, cudaStream_t stream) {
  constexpr int MT = 2;
  const size_t smem = (size_t)NT * 8 * kTiledXStride * sizeof(__half);
  auto kernel = qlinear_tiled_kernel<CODEC, MT, NT>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid((unsigned)plan.grid_x, (unsigned)plan.splits);
  kernel<<<grid, kTiledWarps * 32, smem, stream>>>(args);
  return cudaGetLastError();
}

cudaError_t launch_qlinear_reduce(const float* scratch, int splits, int vpad, int vectors, int rows, int rows_padded,
                                  const float* bias, const float* residual, int epilogue, float* out, __half* out_xh,
                                  cudaStream_t stream, int xh_nv) {
  const int out_cols = epilogue == ETC_EPILOGUE_SWIGLU ? rows / 2 : rows;
  const int64_t total = (int64_t)vectors * out_cols;
  if (total == 0) return cudaSuccess;
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8);
  return launch_chained(qlinear_reduce_kernel, dim3(grid), dim3(256), 0, stream, scratch, splits, vpad, vectors, rows, rows_padded, bias, residual,
                        epilogue, out, vectors <= xh_nv ? out_xh : (__half*)nullptr, xh_nv);
}

// Scratch layout of the tcgen05 path: [xh8 activations, rounded to 256 B][split-K partials].
static size_t umma_xh_region(const UmmaPlan& p) { return (p.xh_bytes + 255) & ~(size_t)255; }

static size_t stream_xh_region(const StreamPlan& p) { return (p.xh_bytes + 255) & ~(size_t)255; }

size_t tiled_scratch_bytes(const TiledWeight& w, int64_t vectors, int sm_count) {
  if (w.layout == kLayoutStream256) {
    size_t need = 0;
    for (int64_t v0 = 0; v0 < vectors; v0 += kStreamMaxVectors) {
      const StreamPlan p = plan_stream(w, std::min<int64_t>(kStreamMaxVectors, vectors - v0), sm_count);
      need = std::max(need, stream_xh_region(p) + p.partial_bytes);
    }
    return need;
  }
  if (w.layout == kLayoutUmma128 && w.counters && vectors <= mv_max_vectors()) {
    const MvPlan p = plan_mv(w, vectors, sm_count);
    return p.xh_bytes + p.partial_bytes;
  }
  if (w.layout == kLayoutUmma128) {
    size_t need = 0;
    for (int64_t v0 = 0; v0 < vectors; v0 += 256) {
      const UmmaPlan p = plan_umma(w, std::min<int64_t>(256, vectors - v0), sm_count);
      need = std::max(need, umma_xh_region(p) + p.scratch_bytes);
    }
    return need;
  }
  return plan_tiled(w, vectors, sm_count).scratch_bytes;
}

cudaError_t launch_qlinear_tiled(const TiledWeight& w, const float* x, int64_t vectors, const float* bias,
                                 const float* residual, int epilogue, float* out, void* scratch, DeviceStatus* status,
                                 int sm_count, cudaStream_t stream, int* launches, const __half* xh_ready, __half* out_xh, int xh_nv) {
  if (w.layout == kLayoutStream256) {
    size_t xh_region = 0;
    for (int64_t v0 = 0; v0 < vectors; v0 += kStreamMaxVectors)
      xh_region = std::max(xh_region, stream_xh_region(plan_stream(w, std::min<int64_t>(kStreamMaxVectors, vectors - v0), sm_count)));
    if (xh_nv != 32) { xh_ready = nullptr; out_xh = nullptr; }  // this layout hands activations over for up to 32 vectors only
    return launch_qlinear_stream(w, x, xh_ready, vectors, bias, residual, epilogue, out, out_xh, reinterpret_cast<__half*>(scratch),
                                 reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + xh_region), status, sm_count, stream,
                                 launches);
  }
  if (w.layout == kLayoutUmma128 && w.counters && vectors <= mv_max_vectors())
    return launch_qlinear_mv(w, x, xh_ready, vectors, bias, residual, epilogue, out, out_xh, scratch, status, sm_count, stream,
                             launches, xh_nv);
  if (w.layout == kLayoutUmma128) {
    // the xh8 region is sized for the widest pass of this call
    size_t xh_region = 0;
    for (int64_t v0 = 0; v0 < vectors; v0 += 256)
      xh_region = std::max(xh_region, umma_xh_region(plan_umma(w, std::min<int64_t>(256, vectors - v0), sm_count)));
    return launch_qlinear_umma(w, x, xh_ready, vectors, bias, residual, epilogue, out, out_xh, reinterpret_cast<__half*>(scratch),
                               reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + xh_region), status, sm_count, stream,
                               launches, xh_nv);
  }
  return launch_qlinear_mma16(w, x, vectors, bias, residual, epilogue, out, reinterpret_cast<float*>(scratch), sm_count, stream,
                              launches);
}

cudaError_t launch_qlinear_mma16(const TiledWeight& w, const float* x, int64_t vectors, const float* bias,
                                 const float* residual, int epilogue, float* out, float* scratch, int sm_count,
                                 cudaStream_t stream, int* launches) {
  const int out_cols = (int)(epilogue == ETC_EPILOGUE_SWIGLU ? w.rows / 2 : w.rows);
  for (int64_t v0 = 0; v0 < vectors; v0 += 32) {
    const int64_t chunk = std::min<int64_t>(32, vectors - v0);
    const TiledPlan plan = plan_tiled(w, chunk, sm_count);
    TiledArgs args;
    args.quants = w.quants;
    args.scales = w.scales;
    args.x = x + v0 * w.columns;
    args.bias = bias;
    args.residual = residual ? residual + v0 * out_cols : nullptr;
    args.out = out + v0 * out_cols;
    args.scratch = scratch;
    args.vectors = (int)chunk;
    args.rows = (int)w.rows;
    args.rows_padded = (int)w.rows_padded;
    args.K = (int)w.columns;
    args.row_tiles = (int)(w.rows_padded / 16);
    args.units = (int)(w.columns / (w.codec == kQ4_0 ? 64 : 32));
    args.units_per_split = (args.units + plan.splits - 1) / plan.splits;
    args.epilogue = epilogue;
    cudaError_t e;
    if (w.codec == kQ4_0) {
      e = plan.nt == 1 ? launch_tiled_pass<kQ4_0, 1>(w, plan, args, stream)
          : plan.nt == 2 ? launch_tiled_pass<kQ4_0, 2>(w, plan, args, stream)
                         : launch_tiled_pass<kQ4_0, 4>(w, plan, args, stream);
    } else if (w.codec == kQ8_0) {
      e = plan.nt == 1 ? launch_tiled_pass<kQ8_0, 1>(w, plan, args, stream)
          : plan.nt == 2 ? launch_tiled_pass<kQ8_0, 2>(w, plan, args, stream)
                         : launch_tiled_pass<kQ8_0, 4>(w, plan, args, stream);
    } else {
      return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
    if (plan.splits > 1) {
      const int64_t total = chunk * out_cols;
      const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8);
      qlinear_reduce_kernel<<<grid, 256, 0, stream>>>(scratch, plan.splits, plan.nt * 8, (int)chunk, (int)w.rows,
                                                      (int)w.rows_padded, bias, args.residual, epilogue, args.out, nullptr, 32);
      e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      if (launches) ++*launches;
    }
  }
  return cudaSuccess;
}

}  // namespace etc
