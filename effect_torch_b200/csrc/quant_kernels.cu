// Block-quantized weight kernels for sm_100a: dequantise, quantise, the generic (any codec, raw
// GGUF layout) linear, the row-gather embedding, the split-K sum of the tcgen05 linear and the
// front end that routes a tiled linear to the matvec kernel (qlinear_mv.cu, up to 16 vectors) or
// to the tcgen05 kernel (qlinear_umma.cu).
//
// Replaces crates/runtime-cpu/src/quantized.rs (decode_block :90, linear_into :419,
// embedding_into :546) of the reference for the CUDA backend.
#include <cuda_fp16.h>

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
// Tiled (128-row) weights: repack front end, split-K sum, dispatch.
// ============================================================================================
cudaError_t launch_repack(const TiledWeight& w, const RepackParts& parts, cudaStream_t stream) { return launch_repack_umma(w, parts, stream); }

__device__ __forceinline__ float silu_tanh_form(float x) { return x * (tanhf(x * 0.5f) * 0.5f + 0.5f); }

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

size_t tiled_scratch_bytes(const TiledWeight& w, int64_t vectors, int sm_count) {
  if (w.counters && vectors <= mv_max_vectors()) {
    const MvPlan p = plan_mv(w, vectors, sm_count);
    return p.xh_bytes + p.partial_bytes;
  }
  const UmmaPlan p = plan_umma(w, vectors, sm_count);
  return umma_xh_region(p) + p.scratch_bytes;
}

cudaError_t launch_qlinear_tiled(const TiledWeight& w, const float* x, int64_t vectors, const float* bias,
                                 const float* residual, int epilogue, float* out, void* scratch, DeviceStatus* status,
                                 int sm_count, cudaStream_t stream, int* launches, const __half* xh_ready, __half* out_xh, int xh_nv,
                                 DeferredSum* defer) {
  if (defer) *defer = DeferredSum();
  if (w.counters && vectors <= mv_max_vectors())
    return launch_qlinear_mv(w, x, xh_ready, vectors, bias, residual, epilogue, out, out_xh, scratch, status, sm_count, stream,
                             launches, xh_nv);
  const size_t xh_region = umma_xh_region(plan_umma(w, vectors, sm_count));  // f16 activations of every chunk, then the partials
  return launch_qlinear_umma(w, x, xh_ready, vectors, bias, residual, epilogue, out, out_xh, reinterpret_cast<__half*>(scratch),
                             reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + xh_region), status, sm_count, stream,
                             launches, xh_nv, defer);
}

}  // namespace etc
