// Dense and elementwise kernels of the decode graph for sm_100a: exact-order dense linear,
// RMSNorm, RoPE, SwiGLU, residual add, greedy argmax, dense embedding gather and the layout
// shuffles around attention. All are HBM/latency-bound single-pass kernels.
//
// Replaces, for the CUDA backend: crates/runtime-cpu/src/matmul.rs:192-231 (naive_into),
// crates/runtime-cpu/src/composed.rs:1457-1487 (rms_norm_forward_into_impl) and :2683-2729
// (rotary_forward_into_impl), the FusedElementwise regions evaluating
// packages/core/src/Tensor.ts:1240-1245,1537-1540 (sigmoid/silu), and the greedy branch of
// crates/runtime/src/sampling.rs:88-105.
#include <cuda_fp16.h>

#include <algorithm>

#include "chain.cuh"
#include "kernels.h"

namespace etc {

// --------------------------------------------------------------------------------------------
// Dense linear, bit-exact with the reference: every output element is one sequential fmaf chain
// over k (out = fma(x[m,k], W[n,k], out)). A CTA computes 32 outputs x 8 input rows; W is staged
// 32 columns at a time through shared memory so global reads stay coalesced.
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ x, int64_t m, int64_t k,
                                                         const float* __restrict__ w, int64_t n,
                                                         const float* __restrict__ bias, float* __restrict__ out) {
  __shared__ float ws[32][33];
  __shared__ float xs[8][32];
  const int tx = threadIdx.x, ty = threadIdx.y;  // tx: output column within tile, ty: input row within tile
  const int64_t n0 = (int64_t)blockIdx.x * 32, m0 = (int64_t)blockIdx.y * 8;
  float acc = 0.0f;
  for (int64_t k0 = 0; k0 < k; k0 += 32) {
    // W tile: rows n0..n0+31, columns k0..k0+31 (coalesced along k)
    for (int r = ty; r < 32; r += 8) {
      const int64_t nn = n0 + r, kk = k0 + tx;
      ws[r][tx] = (nn < n && kk < k) ? w[nn * k + kk] : 0.0f;
    }
    {
      const int64_t mm = m0 + ty, kk = k0 + tx;
      xs[ty][tx] = (mm < m && kk < k) ? x[mm * k + kk] : 0.0f;
    }
    __syncthreads();
    const int len = (int)min((int64_t)32, k - k0);
    for (int kk = 0; kk < len; ++kk) acc = fmaf(xs[ty][kk], ws[tx][kk], acc);
    __syncthreads();
  }
  const int64_t mm = m0 + ty, nn = n0 + tx;
  if (mm < m && nn < n) out[mm * n + nn] = bias ? acc + bias[nn] : acc;
}

cudaError_t launch_linear_f32(const float* x, int64_t m, int64_t k, const float* w, int64_t n, const float* bias,
                              float* out, cudaStream_t stream) {
  if (m == 0 || n == 0) return cudaSuccess;
  dim3 block(32, 8), grid((unsigned)((n + 31) / 32), (unsigned)((m + 7) / 8));
  linear_f32_kernel<<<grid, block, 0, stream>>>(x, m, k, w, n, bias, out);
  return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------
// RMSNorm: one CTA per row, sum of squares and the scaling in f64 like the reference
// (scale = 1/sqrt(ms/n + eps); out = f32(x * scale * w)). The f64 block reduction is a tree, so
// the sum can differ from the reference's sequential sum in the last f64 bits only.
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                      double eps, int64_t n, float* __restrict__ out) {
  __shared__ double partial[8];
  __shared__ double scale_s;
  const float* src = x + (int64_t)blockIdx.x * n;
  double sum = 0.0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const double v = (double)src[i];
    sum += v * v;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += partial[i];
    scale_s = 1.0 / sqrt(total / (double)n + eps);
  }
  __syncthreads();
  const double scale = scale_s;
  float* dst = out + (int64_t)blockIdx.x * n;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const double w = weight ? (double)weight[i] : 1.0;
    dst[i] = (float)(__dmul_rn(__dmul_rn((double)src[i], scale), w));
  }
}

// Single-pass variant for n <= 8192, n % 4 == 0: the row stays in registers between the reduction and the
// scaling (same f64 arithmetic). XH = true stores the result as f16 in [n/8][32][8] order (row < 32), the
// B-operand layout of the tcgen05 linear, instead of f32 row-major.
// SUM = true first adds a projection's split-K partials (summed in split order) onto the row and stores it back: the
// residual update the projection's own sum kernel would have done.
template <bool XH, bool SUM, int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_rows_kernel(const float* x, const float* __restrict__ weight,
                                                               double eps, int n, float* __restrict__ out, __half* __restrict__ out_xh,
                                                               int xh_nv, DeferredSum sum_in, float* x_out) {
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  constexpr int ITEMS = 2048 / THREADS;  // float4 chunks per thread: rows of up to 8192 values
  const int chunks = n / 4;
  float4 w[ITEMS];
  auto load_weight = [&]() {
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      const int c = threadIdx.x + THREADS * j;
      w[j] = weight && c < chunks ? reinterpret_cast<const float4*>(weight)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
    }
  };
  // The f16 hand-off forms are launched by the decoder alone, whose norm weights no kernel writes after the load: they
  // are fetched while the kernel before this one is still running. The plain form may be given a weight that the
  // previous kernel of the stream produced, and reads it after the wait.
  if (XH) load_weight();
  chain_wait();
  if (!XH) load_weight();
  __shared__ double partial[THREADS / 32];
  const int row = blockIdx.x;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)row * n);
  float4 v[ITEMS];
  double sum = 0.0;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const int c = threadIdx.x + THREADS * j;
    v[j] = c < chunks ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (SUM && c < chunks) {
      // all splits' loads are independent: issued together, added in split order
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const float* base = sum_in.partials + (size_t)row * sum_in.rows_padded + 4 * c;
      const size_t split_stride = (size_t)sum_in.vpad * sum_in.rows_padded;
#pragma unroll 4
      for (int s = 0; s < sum_in.splits; ++s) {
        const float4 p = *reinterpret_cast<const float4*>(base + (size_t)s * split_stride);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
      }
      v[j].x += acc.x; v[j].y += acc.y; v[j].z += acc.z; v[j].w += acc.w;
      reinterpret_cast<float4*>(x_out + (size_t)row * n)[c] = v[j];
    }
    sum += (double)v[j].x * (double)v[j].x + (double)v[j].y * (double)v[j].y + (double)v[j].z * (double)v[j].z +
           (double)v[j].w * (double)v[j].w;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
  __syncthreads();
  // every thread adds the warps' sums in the same order and takes the reciprocal root itself: one barrier, no hand-over
  double total = 0.0;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total += partial[i];
  const double scale = 1.0 / sqrt(total / (double)n + eps);
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const int c = threadIdx.x + THREADS * j;
    if (c >= chunks) continue;
    const float r0 = (float)__dmul_rn(__dmul_rn((double)v[j].x, scale), (double)w[j].x);
    const float r1 = (float)__dmul_rn(__dmul_rn((double)v[j].y, scale), (double)w[j].y);
    const float r2 = (float)__dmul_rn(__dmul_rn((double)v[j].z, scale), (double)w[j].z);
    const float r3 = (float)__dmul_rn(__dmul_rn((double)v[j].w, scale), (double)w[j].w);
    if (XH) {
      auto sat = [](float f) { return fminf(fmaxf(f, -65504.f), 65504.f); };
      __half2 h01 = __floats2half2_rn(sat(r0), sat(r1)), h23 = __floats2half2_rn(sat(r2), sat(r3));
      const int k = 4 * c;
      uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&h01), *reinterpret_cast<uint32_t*>(&h23));
      *reinterpret_cast<uint2*>(out_xh + ((size_t)(k >> 3) * xh_nv + row) * 8 + (k & 7)) = packed;
    } else {
      reinterpret_cast<float4*>(out + (size_t)row * n)[c] = make_float4(r0, r1, r2, r3);
    }
  }
}

static bool rmsnorm_fast_ok(const float* x, const float* weight, int64_t n) {
  return n % 4 == 0 && n <= 8192 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)weight % 16) == 0;
}

cudaError_t launch_rmsnorm(const float* x, const float* weight, double eps, int64_t rows, int64_t n, float* out,
                           cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if (rmsnorm_fast_ok(x, weight, n) && ((uintptr_t)out % 16) == 0)
    return launch_chained(rmsnorm_rows_kernel<false, false, 256>, dim3((unsigned)rows), dim3(256), 0, stream, x, weight, eps, (int)n, out, (__half*)nullptr, 32,
                          DeferredSum(), (float*)nullptr);
  else
    rmsnorm_kernel<<<(unsigned)rows, 256, 0, stream>>>(x, weight, eps, n, out);
  return cudaGetLastError();
}

cudaError_t launch_rmsnorm_xh8(const float* x, const float* weight, double eps, int64_t rows, int64_t n, __half* out_xh,
                               cudaStream_t stream, int xh_nv) {
  if (rows == 0) return cudaSuccess;
  if (rows > xh_nv || n % 8 != 0 || !rmsnorm_fast_ok(x, weight, n)) return cudaErrorInvalidValue;
  return launch_chained(rmsnorm_rows_kernel<true, false, 256>, dim3((unsigned)rows), dim3(256), 0, stream, x, weight, eps, (int)n, (float*)nullptr, out_xh, xh_nv,
                        DeferredSum(), (float*)nullptr);
}

cudaError_t launch_sum_rmsnorm_xh8(float* x, const DeferredSum& sum, const float* weight, double eps, int64_t rows, int64_t n,
                                   __half* out_xh, cudaStream_t stream, int xh_nv) {
  if (rows == 0) return cudaSuccess;
  if (rows > xh_nv || n % 8 != 0 || !rmsnorm_fast_ok(x, weight, n) || sum.splits <= 0 || sum.rows_padded % 4 != 0 || rows > sum.vpad)
    return cudaErrorInvalidValue;
  return launch_chained(rmsnorm_rows_kernel<true, true, 1024>, dim3((unsigned)rows), dim3(1024), 0, stream, (const float*)x, weight, eps, (int)n,
                        (float*)nullptr, out_xh, xh_nv, sum, x);
}

// --------------------------------------------------------------------------------------------
// RoPE on [batch, heads, steps, head_dim] with per-lane cursor offsets. inv_freq[j] =
// theta^(-2j/D) is precomputed on the host in f64 with the same pow() the reference calls;
// angle, sin/cos and the rotation are f64, results are rounded to f32 once.
// --------------------------------------------------------------------------------------------
__global__ void rope_kernel(const float* __restrict__ x, const int64_t* __restrict__ offsets, int64_t n_offsets,
                            const double* __restrict__ inv_freq, int layout, int64_t batch, int64_t heads,
                            int64_t steps, int64_t head_dim, float* __restrict__ out) {
  const int64_t half = head_dim / 2;
  const int64_t total = batch * heads * steps * half;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t j = idx % half;
    const int64_t row_step = idx / half;  // (batch*heads + head)*steps + step
    const int64_t step = row_step % steps;
    const int64_t b = row_step / (steps * heads);
    const int64_t offset = n_offsets == 1 ? offsets[0] : offsets[b];
    const double angle = (double)(offset + step) * inv_freq[j];
    double s, c;
    sincos(angle, &s, &c);
    const int64_t base = row_step * head_dim;
    const int64_t i0 = layout == 0 ? base + j : base + 2 * j;
    const int64_t i1 = layout == 0 ? base + half + j : base + 2 * j + 1;
    const double first = (double)x[i0], second = (double)x[i1];
    out[i0] = (float)__dsub_rn(__dmul_rn(first, c), __dmul_rn(second, s));
    out[i1] = (float)__dadd_rn(__dmul_rn(second, c), __dmul_rn(first, s));
  }
}

cudaError_t launch_rope(const float* x, const int64_t* offsets, int64_t n_offsets, const double* inv_freq, int layout,
                        int64_t batch, int64_t heads, int64_t steps, int64_t head_dim, float* out, cudaStream_t stream) {
  const int64_t total = batch * heads * steps * (head_dim / 2);
  if (total == 0) return cudaSuccess;
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8);
  rope_kernel<<<grid, 256, 0, stream>>>(x, offsets, n_offsets, inv_freq, layout, batch, heads, steps, head_dim, out);
  return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------
// silu(gate) * up with the reference's definition sigmoid(x) = tanh(x/2)/2 + 1/2, evaluated in
// f32 like the reference's expression interpreter. exact != 0 takes tanh in f64 and rounds, which
// tracks a correctly rounded tanhf more closely than the device tanhf.
// --------------------------------------------------------------------------------------------
__global__ void swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, int64_t n,
                              float* __restrict__ out, int exact) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float g = gate[i];
    const float half_g = __fdiv_rn(g, 2.0f);
    const float th = exact ? (float)tanh((double)half_g) : tanhf(half_g);
    const float sig = __fadd_rn(__fdiv_rn(th, 2.0f), 0.5f);
    out[i] = __fmul_rn(__fmul_rn(g, sig), up[i]);
  }
}
cudaError_t launch_swiglu(const float* gate, const float* up, int64_t n, float* out, int exact, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const unsigned grid = (unsigned)std::min<int64_t>((n + 255) / 256, 148 * 8);
  swiglu_kernel<<<grid, 256, 0, stream>>>(gate, up, n, out, exact);
  return cudaGetLastError();
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t n, float* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = __fadd_rn(a[i], b[i]);
}
cudaError_t launch_add(const float* a, const float* b, int64_t n, float* out, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const unsigned grid = (unsigned)std::min<int64_t>((n + 255) / 256, 148 * 8);
  add_kernel<<<grid, 256, 0, stream>>>(a, b, n, out);
  return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------
// Greedy argmax per row: the first index of the maximum (strict >, so the lowest index wins
// ties); a non-finite logit raises the status word with its index.
// --------------------------------------------------------------------------------------------
// `picks` (optional): the row's (best logit bits, index_base + index) pair, for the exchange between the ranks of a
// vocabulary-parallel head.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int64_t vocab,
                                                      uint32_t* __restrict__ tokens, DeviceStatus* status, uint2* picks,
                                                      uint32_t index_base) {
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  chain_wait();
  __shared__ float best_v[32];
  __shared__ long long best_i[32];
  __shared__ long long bad_s[32];
  const float* row = logits + (int64_t)blockIdx.x * vocab;
  float best = -INFINITY;
  long long arg = 0x7fffffffffffffffll;
  long long bad = 0x7fffffffffffffffll;
  auto take = [&](float v, int64_t i) {
    if (!isfinite(v)) bad = min(bad, (long long)i);
    if (v > best) { best = v; arg = i; }
  };
  int64_t head = 0;
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // 16-byte loads, four in flight per thread; a thread's indices still ascend, so strict > keeps the lowest index
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int64_t n4 = vocab >> 2;
    int64_t i = threadIdx.x;
    for (; i + 3 * (int64_t)blockDim.x < n4; i += 4 * (int64_t)blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = row4[i + u * (int64_t)blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t base = (i + u * (int64_t)blockDim.x) << 2;
        take(v[u].x, base); take(v[u].y, base + 1); take(v[u].z, base + 2); take(v[u].w, base + 3);
      }
    }
    for (; i < n4; i += blockDim.x) {
      const float4 v = row4[i];
      take(v.x, i << 2); take(v.y, (i << 2) + 1); take(v.z, (i << 2) + 2); take(v.w, (i << 2) + 3);
    }
    head = vocab;
  }
  for (int64_t i = head + threadIdx.x; i < vocab; i += blockDim.x) take(row[i], i);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const long long oi = __shfl_xor_sync(0xffffffffu, arg, off);
    const long long ob = __shfl_xor_sync(0xffffffffu, bad, off);
    if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
    bad = min(bad, ob);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { best_v[warp] = best; best_i[warp] = arg; bad_s[warp] = bad; }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = blockDim.x >> 5;
    best = lane < nwarps ? best_v[lane] : -INFINITY;
    arg = lane < nwarps ? best_i[lane] : 0x7fffffffffffffffll;
    bad = lane < nwarps ? bad_s[lane] : 0x7fffffffffffffffll;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, off);
      const long long oi = __shfl_xor_sync(0xffffffffu, arg, off);
      const long long ob = __shfl_xor_sync(0xffffffffu, bad, off);
      if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
      bad = min(bad, ob);
    }
    if (lane == 0) {
      // a row of only -inf keeps index 0 like the reference's loop would before it errors
      tokens[blockIdx.x] = index_base + (arg == 0x7fffffffffffffffll ? 0u : (uint32_t)arg);
      if (picks) picks[blockIdx.x] = make_uint2(__float_as_uint(best), index_base + (arg == 0x7fffffffffffffffll ? 0u : (uint32_t)arg));
      if (bad != 0x7fffffffffffffffll && atomicCAS(&status->code, kStatusNone, kStatusNonFiniteLogit) == kStatusNone) {
        status->value = bad;
        status->bound = vocab;
      }
    }
  }
}
cudaError_t launch_argmax(const float* logits, int64_t rows, int64_t vocab, uint32_t* tokens, DeviceStatus* status,
                          cudaStream_t stream, uint2* picks, uint32_t index_base) {
  if (rows == 0) return cudaSuccess;
  return launch_chained(argmax_kernel, dim3((unsigned)rows), dim3(1024), 0, stream, logits, vocab, tokens, status, picks, index_base);
}

// Dense f32 embedding gather with the same bounds rule as the quantized embedding.
template <typename Index>
__global__ void embedding_f32_kernel(const Index* __restrict__ indexes, int64_t count, const float* __restrict__ table,
                                     int64_t rows, int64_t columns, float* __restrict__ out, DeviceStatus* status) {
  chain_release();  // the next kernel of the step may be scheduled; it waits for this one before touching memory
  chain_wait();
  const int64_t i = blockIdx.y;
  const long long row = (long long)indexes[i];
  if (row < 0 || row >= rows) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && atomicCAS(&status->code, kStatusNone, kStatusIndexOutOfRange) == kStatusNone) {
      status->value = row;
      status->bound = rows;
    }
    return;
  }
  for (int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; c < columns; c += (int64_t)gridDim.x * blockDim.x)
    out[i * columns + c] = table[row * columns + c];
}
cudaError_t launch_embedding_f32(const void* indexes, int index_is_i64, int64_t count, const float* table, int64_t rows,
                                 int64_t columns, float* out, DeviceStatus* status, cudaStream_t stream) {
  if (count == 0) return cudaSuccess;
  dim3 grid((unsigned)std::min<int64_t>((columns + 255) / 256, 32), (unsigned)count);
  if (index_is_i64)
    return launch_chained(embedding_f32_kernel<long long>, grid, dim3(256), 0, stream, (const long long*)indexes, count, table, rows, columns, out, status);
  else
    return launch_chained(embedding_f32_kernel<unsigned int>, grid, dim3(256), 0, stream, (const unsigned int*)indexes, count, table, rows, columns, out, status);
  return cudaGetLastError();
}

// [B,T,H*D] (row stride src_row_stride floats) -> [B,H,T,D]
__global__ void heads_first_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t B, int64_t T, int64_t H,
                                   int64_t D, int64_t src_row_stride) {
  const int64_t total = B * H * T * D;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t d = idx % D, t = (idx / D) % T, h = (idx / (D * T)) % H, b = idx / (D * T * H);
    dst[idx] = src[(b * T + t) * src_row_stride + h * D + d];
  }
}
cudaError_t launch_heads_first(const float* src, float* dst, int64_t B, int64_t T, int64_t H, int64_t D,
                               int64_t src_row_stride, cudaStream_t stream) {
  const int64_t total = B * H * T * D;
  if (total == 0) return cudaSuccess;
  heads_first_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8), 256, 0, stream>>>(src, dst, B, T, H, D, src_row_stride);
  return cudaGetLastError();
}
// [B,H,T,D] -> [B,T,H*D]
__global__ void heads_last_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t B, int64_t T, int64_t H,
                                  int64_t D) {
  const int64_t total = B * H * T * D;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t d = idx % D, h = (idx / D) % H, t = (idx / (D * H)) % T, b = idx / (D * H * T);
    dst[idx] = src[((b * H + h) * T + t) * D + d];
  }
}
cudaError_t launch_heads_last(const float* src, float* dst, int64_t B, int64_t T, int64_t H, int64_t D, cudaStream_t stream) {
  const int64_t total = B * H * T * D;
  if (total == 0) return cudaSuccess;
  heads_last_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8), 256, 0, stream>>>(src, dst, B, T, H, D);
  return cudaGetLastError();
}

// LastTokenRow (crates/runtime-cpu/src/napi/mod.rs:3053-3075) for every lane at once.
__global__ void last_token_rows_kernel(const float* __restrict__ src, int64_t lanes, int64_t steps, int64_t width,
                                       int64_t advance, float* __restrict__ out) {
  const int64_t total = lanes * width;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t lane = idx / width, c = idx - lane * width;
    out[idx] = src[(lane * steps + (advance - 1)) * width + c];
  }
}
cudaError_t launch_last_token_rows(const float* src, int64_t lanes, int64_t steps, int64_t width, int64_t advance,
                                   float* out, cudaStream_t stream) {
  const int64_t total = lanes * width;
  if (total == 0) return cudaSuccess;
  last_token_rows_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8), 256, 0, stream>>>(src, lanes, steps, width, advance, out);
  return cudaGetLastError();
}

}  // namespace etc
