// TEST INFRASTRUCTURE ONLY — CPU restatement of effect-torch's reference CPU backend
// for the compiled-inference hot path (paged-KV batched decode over block-quantized
// weights). Nothing in the product library links or calls this file; only the test
// suite, the smoke check and the benchmark's CPU-baseline leg load it.
//
// Every routine restates, in its own code, the arithmetic and the loop/accumulation
// order of the reference routine named in its comment (paths are relative to the
// reference project root). Parity status:
//   * K-quant decoders, quantized linear/embedding, paged attention, slab tiers, block
//     allocator, prefix hashing, greedy sampling, RMSNorm, RoPE, dense matmul: PINNED by
//     the reference's own golden vectors (tests/test_oracle_golden.py lists each one).
//   * Q4_0 / Q8_0 codecs and the weight quantizer: PARITY UNPINNED. The reference has
//     neither codec (its GGUF parser rejects their type codes); they are defined here
//     from the published block format (32 values per block; an f16 scale followed by 16
//     nibble bytes, value = scale * (code - 8), low nibbles are values 0..15 and high
//     nibbles values 16..31; resp. an f16 scale followed by 32 int8, value = scale * code).
//
// Build: make -C oracle   (g++ -O2 -march=x86-64-v3 -ffp-contract=off: the reference never fuses a
// multiply with an add unless it calls mul_add explicitly, so contraction is disabled
// and std::fma is used exactly where the reference uses mul_add).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

// ----------------------------------------------------------------------------------
// Scalar conversions (half 2.7.1 semantics: IEEE round-to-nearest-even both ways).
// ----------------------------------------------------------------------------------
static inline float f16_bits_to_f32(uint16_t bits) {
  _Float16 h;
  std::memcpy(&h, &bits, 2);
  return (float)h;
}
static inline uint16_t f32_to_f16_bits(float value) {
  _Float16 h = (_Float16)value;
  uint16_t bits;
  std::memcpy(&bits, &h, 2);
  return bits;
}
static inline float bf16_bits_to_f32(uint16_t bits) {
  uint32_t wide = (uint32_t)bits << 16;
  float value;
  std::memcpy(&value, &wide, 4);
  return value;
}
static inline uint16_t f32_to_bf16_bits(float value) {
  uint32_t x;
  std::memcpy(&x, &value, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u);  // quiet NaN
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7fffu + lsb;
  return (uint16_t)(x >> 16);
}

ORC_API uint16_t orc_f32_to_f16(float v) { return f32_to_f16_bits(v); }
ORC_API float orc_f16_to_f32(uint16_t v) { return f16_bits_to_f32(v); }
ORC_API uint16_t orc_f32_to_bf16(float v) { return f32_to_bf16_bits(v); }
ORC_API float orc_bf16_to_f32(uint16_t v) { return bf16_bits_to_f32(v); }

// ----------------------------------------------------------------------------------
// Block codecs. Codec ids are the GGML tensor type codes the GGUF catalog stores
// (crates/runtime/src/gguf.rs:279-291 for 10..14; 2 and 8 are this build's additions).
// ----------------------------------------------------------------------------------
enum { ORC_Q4_0 = 2, ORC_Q8_0 = 8, ORC_Q2_K = 10, ORC_Q3_K = 11, ORC_Q4_K = 12, ORC_Q5_K = 13, ORC_Q6_K = 14 };

ORC_API int orc_block_values(int codec) {
  switch (codec) {
    case ORC_Q4_0: case ORC_Q8_0: return 32;
    case ORC_Q2_K: case ORC_Q3_K: case ORC_Q4_K: case ORC_Q5_K: case ORC_Q6_K: return 256;
    default: return 0;
  }
}

// crates/runtime-cpu/src/quantized.rs:60-68 (K-quants); 18 / 34 from the published block format.
ORC_API int orc_block_bytes(int codec) {
  switch (codec) {
    case ORC_Q4_0: return 18;
    case ORC_Q8_0: return 34;
    case ORC_Q2_K: return 84;
    case ORC_Q3_K: return 110;
    case ORC_Q4_K: return 144;
    case ORC_Q5_K: return 176;
    case ORC_Q6_K: return 210;
    default: return 0;
  }
}

// crates/runtime/src/gguf.rs:245-250: columns must be a whole number of blocks.
ORC_API long long orc_encoded_row_bytes(int codec, long long columns) {
  int values = orc_block_values(codec);
  if (values == 0 || columns < 0 || columns % values != 0) return -1;
  return columns / values * orc_block_bytes(codec);
}

static inline float fp16_at(const uint8_t* block, int offset) {  // quantized.rs:71-73
  return f16_bits_to_f32((uint16_t)(block[offset] | (block[offset + 1] << 8)));
}

// quantized.rs:77-86 — 6-bit (scale, min) pair of group `index` in the 12-byte field.
static inline void scale_min_k4(int index, const uint8_t* scales, uint8_t* scale, uint8_t* min) {
  if (index < 4) {
    *scale = scales[index] & 63;
    *min = scales[index + 4] & 63;
  } else {
    *scale = (uint8_t)((scales[index + 4] & 0x0f) | ((scales[index - 4] >> 6) << 4));
    *min = (uint8_t)((scales[index + 4] >> 4) | ((scales[index] >> 6) << 4));
  }
}

static void decode_q2_k(const uint8_t* b, float* out) {  // quantized.rs:117-138
  const uint8_t* scales = b;
  const uint8_t* quants = b + 16;
  const float d = fp16_at(b, 80), dmin = fp16_at(b, 82);
  int group = 0;
  for (int half = 0; half < 2; ++half) {
    const uint8_t* q = quants + half * 32;
    for (int shift = 0; shift < 8; shift += 2) {
      for (int q_offset = 0; q_offset < 32; q_offset += 16) {
        const uint8_t sc = scales[group];
        const float dl = d * (float)(sc & 0x0f);
        const float ml = dmin * (float)(sc >> 4);
        for (int i = 0; i < 16; ++i) out[group * 16 + i] = dl * (float)((q[q_offset + i] >> shift) & 3) - ml;
        ++group;
      }
    }
  }
}

static void decode_q3_k(const uint8_t* b, float* out) {  // quantized.rs:142-176
  const uint8_t* hmask = b;
  const uint8_t* quants = b + 32;
  const uint8_t* packed = b + 96;
  const float d = fp16_at(b, 108);
  int group = 0;
  for (int half = 0; half < 2; ++half) {
    const uint8_t* q = quants + half * 32;
    for (int lane = 0; lane < 4; ++lane) {
      const int shift = lane * 2;
      const uint8_t mask = (uint8_t)(1u << (half * 4 + lane));
      for (int q_offset = 0; q_offset < 32; q_offset += 16) {
        const uint8_t low = group < 8 ? (packed[group] & 0x0f) : (packed[group - 8] >> 4);
        const uint8_t high = (packed[8 + group % 4] >> (2 * (group / 4))) & 3;
        const int scale = (int)(low | (high << 4)) - 32;
        const float dl = d * (float)scale;
        for (int i = 0; i < 16; ++i) {
          const int low_q = (q[q_offset + i] >> shift) & 3;
          const int high_q = (hmask[q_offset + i] & mask) == 0 ? 4 : 0;
          out[group * 16 + i] = dl * (float)(low_q - high_q);
        }
        ++group;
      }
    }
  }
}

static void decode_q4_k(const uint8_t* b, float* out) {  // quantized.rs:180-199
  const float d = fp16_at(b, 0), dmin = fp16_at(b, 2);
  const uint8_t* scales = b + 4;
  const uint8_t* quants = b + 16;
  for (int pair = 0; pair < 4; ++pair) {
    const uint8_t* q = quants + pair * 32;
    for (int side = 0; side < 2; ++side) {
      const int group = pair * 2 + side;
      uint8_t sc, mn;
      scale_min_k4(group, scales, &sc, &mn);
      const float dl = d * (float)sc, ml = dmin * (float)mn;
      for (int i = 0; i < 32; ++i) {
        const uint8_t code = side == 0 ? (q[i] & 0x0f) : (q[i] >> 4);
        out[group * 32 + i] = dl * (float)code - ml;
      }
    }
  }
}

static void decode_q5_k(const uint8_t* b, float* out) {  // quantized.rs:203-234
  const float d = fp16_at(b, 0), dmin = fp16_at(b, 2);
  const uint8_t* scales = b + 4;
  const uint8_t* high = b + 16;
  const uint8_t* low = b + 48;
  for (int pair = 0; pair < 4; ++pair) {
    const uint8_t* ql = low + pair * 32;
    for (int side = 0; side < 2; ++side) {
      const int group = pair * 2 + side;
      const uint8_t mask = (uint8_t)(1u << (pair * 2 + side));
      uint8_t sc, mn;
      scale_min_k4(group, scales, &sc, &mn);
      const float dl = d * (float)sc, ml = dmin * (float)mn;
      for (int i = 0; i < 32; ++i) {
        const uint8_t low_q = side == 0 ? (ql[i] & 0x0f) : (ql[i] >> 4);
        const uint8_t code = (uint8_t)(low_q + ((high[i] & mask) == 0 ? 0 : 16));
        out[group * 32 + i] = dl * (float)code - ml;
      }
    }
  }
}

static void decode_q6_k(const uint8_t* b, float* out) {  // quantized.rs:238-261
  const uint8_t* low = b;
  const uint8_t* high = b + 128;
  const float d = fp16_at(b, 208);
  for (int half = 0; half < 2; ++half) {
    const uint8_t* ql = low + half * 64;
    const uint8_t* qh = high + half * 32;
    for (int i = 0; i < 32; ++i) {
      const int scale_lane = i / 16;
      const uint8_t codes[4] = {
          (uint8_t)((ql[i] & 0x0f) | (((qh[i] >> 0) & 3) << 4)),
          (uint8_t)((ql[i + 32] & 0x0f) | (((qh[i] >> 2) & 3) << 4)),
          (uint8_t)((ql[i] >> 4) | (((qh[i] >> 4) & 3) << 4)),
          (uint8_t)((ql[i + 32] >> 4) | (((qh[i] >> 6) & 3) << 4)),
      };
      for (int quarter = 0; quarter < 4; ++quarter) {
        const int scale_index = half * 8 + scale_lane + quarter * 2;
        const int8_t scale = (int8_t)b[192 + scale_index];
        const int code = (int)codes[quarter] - 32;
        out[half * 128 + quarter * 32 + i] = d * (float)scale * (float)code;
      }
    }
  }
}

// Q4_0 / Q8_0: defined by this build from the published block format (see file header).
static void decode_q4_0(const uint8_t* b, float* out) {
  const float d = fp16_at(b, 0);
  for (int i = 0; i < 16; ++i) {
    out[i] = d * (float)((int)(b[2 + i] & 0x0f) - 8);
    out[i + 16] = d * (float)((int)(b[2 + i] >> 4) - 8);
  }
}
static void decode_q8_0(const uint8_t* b, float* out) {
  const float d = fp16_at(b, 0);
  for (int i = 0; i < 32; ++i) out[i] = d * (float)(int8_t)b[2 + i];
}

// quantized.rs:90-111. Returns 0, or -1 when `len` is not the codec's block size
// (the reference's error text contains "expected").
ORC_API int orc_decode_block(int codec, const uint8_t* block, long long len, float* out) {
  if (orc_block_bytes(codec) == 0 || len != orc_block_bytes(codec)) return -1;
  switch (codec) {
    case ORC_Q4_0: decode_q4_0(block, out); break;
    case ORC_Q8_0: decode_q8_0(block, out); break;
    case ORC_Q2_K: decode_q2_k(block, out); break;
    case ORC_Q3_K: decode_q3_k(block, out); break;
    case ORC_Q4_K: decode_q4_k(block, out); break;
    case ORC_Q5_K: decode_q5_k(block, out); break;
    case ORC_Q6_K: decode_q6_k(block, out); break;
  }
  return 0;
}

// Whole-matrix dequantisation (rows x columns f32). Convenience for tests.
ORC_API int orc_dequantize(int codec, const uint8_t* packed, long long rows, long long columns, float* out) {
  const long long row_bytes = orc_encoded_row_bytes(codec, columns);
  if (row_bytes < 0) return -1;
  const int bv = orc_block_values(codec), bb = orc_block_bytes(codec);
  for (long long r = 0; r < rows; ++r)
    for (long long blk = 0; blk < columns / bv; ++blk)
      orc_decode_block(codec, packed + r * row_bytes + blk * bb, bb, out + r * columns + blk * bv);
  return 0;
}

// Weight quantizers (this build's own; the reference has none).
//   Q4_0: per 32-value block take the element of largest magnitude, signed; scale d = that / -8
//         so the extreme value maps onto code 0 (= -8); store d as f16; code = clamp(floor(x * (1/d)
//         + 8.5), 0, 15) with the unrounded f32 d.  d == 0 -> all codes 8.
//   Q8_0: d = absmax / 127, store as f16; code = round-half-away(x * (1/d)) clamped to +-127 with
//         the unrounded f32 d.
ORC_API void orc_quantize_q4_0(const float* x, long long rows, long long columns, uint8_t* out) {
  const long long blocks = columns / 32;
  for (long long r = 0; r < rows; ++r) {
    for (long long blk = 0; blk < blocks; ++blk) {
      const float* src = x + r * columns + blk * 32;
      uint8_t* dst = out + (r * blocks + blk) * 18;
      float amax = 0.0f, extreme = 0.0f;
      for (int i = 0; i < 32; ++i) {
        const float a = std::fabs(src[i]);
        if (a > amax) { amax = a; extreme = src[i]; }
      }
      const float d = extreme / -8.0f;
      const float inv = d != 0.0f ? 1.0f / d : 0.0f;
      const uint16_t dbits = f32_to_f16_bits(d);
      dst[0] = (uint8_t)(dbits & 0xff);
      dst[1] = (uint8_t)(dbits >> 8);
      for (int i = 0; i < 16; ++i) {
        int lo = (int)std::floor(src[i] * inv + 8.5f);
        int hi = (int)std::floor(src[i + 16] * inv + 8.5f);
        lo = lo < 0 ? 0 : (lo > 15 ? 15 : lo);
        hi = hi < 0 ? 0 : (hi > 15 ? 15 : hi);
        dst[2 + i] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
}

ORC_API void orc_quantize_q8_0(const float* x, long long rows, long long columns, uint8_t* out) {
  const long long blocks = columns / 32;
  for (long long r = 0; r < rows; ++r) {
    for (long long blk = 0; blk < blocks; ++blk) {
      const float* src = x + r * columns + blk * 32;
      uint8_t* dst = out + (r * blocks + blk) * 34;
      float amax = 0.0f;
      for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(src[i]));
      const float d = amax / 127.0f;
      const float inv = d != 0.0f ? 1.0f / d : 0.0f;
      const uint16_t dbits = f32_to_f16_bits(d);
      dst[0] = (uint8_t)(dbits & 0xff);
      dst[1] = (uint8_t)(dbits >> 8);
      for (int i = 0; i < 32; ++i) {
        float q = std::round(src[i] * inv);
        q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
        dst[2 + i] = (uint8_t)(int8_t)q;
      }
    }
  }
}

// ----------------------------------------------------------------------------------
// Quantized linear / embedding.
// ----------------------------------------------------------------------------------

// quantized.rs:419-499 — reference-faithful: vector -> row -> block -> lane, one f32
// accumulator, separate multiply and add, every block re-decoded per input vector, the
// cancellation flag polled per row and per block. Returns 0, or 1 = "operation aborted".
ORC_API int orc_qlinear(int codec, const float* x, long long vectors, long long columns, const uint8_t* packed,
                        long long rows, const float* bias, float* out, const volatile int* cancelled) {
  const long long row_bytes = orc_encoded_row_bytes(codec, columns);
  if (row_bytes < 0) return -1;
  const int bv = orc_block_values(codec), bb = orc_block_bytes(codec);
  const long long blocks = columns / bv;
  float decoded[256];
  for (long long v = 0; v < vectors; ++v) {
    for (long long r = 0; r < rows; ++r) {
      if (cancelled && *cancelled) return 1;
      float sum = 0.0f;
      for (long long blk = 0; blk < blocks; ++blk) {
        if (cancelled && *cancelled) return 1;
        orc_decode_block(codec, packed + r * row_bytes + blk * bb, bb, decoded);
        const float* xin = x + v * columns + blk * bv;
        for (int lane = 0; lane < bv; ++lane) sum += xin[lane] * decoded[lane];
      }
      if (bias) sum += bias[r];
      out[v * rows + r] = sum;
    }
  }
  return 0;
}

// Same arithmetic and the same per-output accumulation order as orc_qlinear (so results are
// bit-identical), but each block is decoded once per row and rows are spread over OpenMP
// threads: the "fair CPU" variant used as the timed multi-core baseline.
ORC_API int orc_qlinear_mt(int codec, const float* x, long long vectors, long long columns, const uint8_t* packed,
                           long long rows, const float* bias, float* out, int threads) {
  const long long row_bytes = orc_encoded_row_bytes(codec, columns);
  if (row_bytes < 0) return -1;
  const int bv = orc_block_values(codec), bb = orc_block_bytes(codec);
  const long long blocks = columns / bv;
  (void)threads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
  {
    std::vector<float> sums((size_t)vectors);
    float decoded[256];
#pragma omp for schedule(static)
    for (long long r = 0; r < rows; ++r) {
      std::fill(sums.begin(), sums.end(), 0.0f);
      for (long long blk = 0; blk < blocks; ++blk) {
        orc_decode_block(codec, packed + r * row_bytes + blk * bb, bb, decoded);
        for (long long v = 0; v < vectors; ++v) {
          const float* xin = x + v * columns + blk * bv;
          float sum = sums[(size_t)v];
          for (int lane = 0; lane < bv; ++lane) sum += xin[lane] * decoded[lane];
          sums[(size_t)v] = sum;
        }
      }
      for (long long v = 0; v < vectors; ++v) out[v * rows + r] = sums[(size_t)v] + (bias ? bias[r] : 0.0f);
    }
  }
  return 0;
}

// quantized.rs:546-616 — i64 indexes (u32 callers widen). Returns 0, or 2 with `bad_index`
// set when an index is negative or >= rows ("index {i} is outside 0..{rows}").
ORC_API int orc_qembedding(int codec, const long long* indexes, long long count, const uint8_t* packed,
                           long long rows, long long columns, float* out, long long* bad_index) {
  const long long row_bytes = orc_encoded_row_bytes(codec, columns);
  if (row_bytes < 0) return -1;
  const int bv = orc_block_values(codec), bb = orc_block_bytes(codec);
  for (long long i = 0; i < count; ++i) {
    const long long row = indexes[i];
    if (row < 0 || row >= rows) {
      if (bad_index) *bad_index = row;
      return 2;
    }
    for (long long blk = 0; blk < columns / bv; ++blk)
      orc_decode_block(codec, packed + row * row_bytes + blk * bb, bb, out + i * columns + blk * bv);
  }
  return 0;
}

// ----------------------------------------------------------------------------------
// Dense kernels.
// ----------------------------------------------------------------------------------

// crates/runtime-cpu/src/matmul.rs:192-231 — C[m,n] = A[m,k] . B[k,n] with explicit strides
// (elements); loop row -> k -> column, c = fma(a, b, c) in f32.
ORC_API void orc_matmul_f32(const float* a, long long a_row, long long a_col, const float* b, long long b_row,
                            long long b_col, float* out, long long m, long long n, long long k) {
  for (long long row = 0; row < m; ++row) {
    float* dst = out + row * n;
    for (long long col = 0; col < n; ++col) dst[col] = 0.0f;
    for (long long inner = 0; inner < k; ++inner) {
      const float left = a[row * a_row + inner * a_col];
      for (long long col = 0; col < n; ++col) dst[col] = std::fma(left, b[inner * b_row + col * b_col], dst[col]);
    }
  }
}

// packages/core/src/Tensor.ts:5242-5245 — linearRows on a dense [N,K] weight is
// matmul(x, transpose(W)): same fma chain with b strides (1, K). `threads` > 1 spreads the
// independent output elements over OpenMP threads without changing any per-output chain.
ORC_API void orc_linear_rows_f32(const float* x, long long m, long long k, const float* w, long long n, float* out,
                                 int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1) collapse(2)
  for (long long row = 0; row < m; ++row) {
    for (long long col = 0; col < n; ++col) {
      float acc = 0.0f;
      const float* xr = x + row * k;
      const float* wr = w + col * k;
      for (long long inner = 0; inner < k; ++inner) acc = std::fma(xr[inner], wr[inner], acc);
      out[row * n + col] = acc;
    }
  }
}

// crates/runtime-cpu/src/composed.rs:1457-1487 — f64 mean of squares in index order,
// scale = 1/sqrt(ms/n + eps), out = f32(x * scale * w) evaluated left to right in f64.
ORC_API void orc_rms_norm(const float* x, const float* weight, double eps, float* out, long long rows, long long n) {
  for (long long row = 0; row < rows; ++row) {
    const float* src = x + row * n;
    double mean_square = 0.0;
    for (long long i = 0; i < n; ++i) {
      const double value = (double)src[i];
      mean_square += value * value;
    }
    const double scale = 1.0 / std::sqrt(mean_square / (double)n + eps);
    for (long long i = 0; i < n; ++i) {
      const double w = weight ? (double)weight[i] : 1.0;
      out[row * n + i] = (float)((double)src[i] * scale * w);
    }
  }
}

// composed.rs:2683-2729 — x is [batch, ..., steps, head_dim]; `rows` = product of all dims but
// the last two; offsets has 1 or `batch` entries; layout 0 = HalfSplit (j, D/2+j),
// 1 = InterleavedPairs (2j, 2j+1); angle = sign * (offset + step) * theta^(-2j/D) in f64.
ORC_API void orc_rotary(const float* x, const long long* offsets, long long n_offsets, double theta, double sign,
                        int layout, float* out, long long batch, long long rows, long long steps, long long head_dim) {
  const long long rows_per_batch = rows / batch;
  const long long half = head_dim / 2;
  for (long long row = 0; row < rows; ++row) {
    const long long batch_index = row / rows_per_batch;
    const long long offset = n_offsets == 1 ? offsets[0] : offsets[batch_index];
    for (long long step = 0; step < steps; ++step) {
      const long long base = (row * steps + step) * head_dim;
      for (long long j = 0; j < half; ++j) {
        const double angle = sign * (double)(offset + step) * std::pow(theta, -2.0 * (double)j / (double)head_dim);
        const double s = std::sin(angle), c = std::cos(angle);
        const long long first_index = layout == 0 ? base + j : base + 2 * j;
        const long long second_index = layout == 0 ? base + half + j : base + 2 * j + 1;
        const double first = (double)x[first_index], second = (double)x[second_index];
        out[first_index] = (float)(first * c - second * s);
        out[second_index] = (float)(second * c + first * s);
      }
    }
  }
}

// packages/core/src/Tensor.ts:1240-1245 and 1537-1540, evaluated by the f32 expression
// interpreter: sigmoid(x) = tanh(x / 2) / 2 + 0.5 ; silu(x) = x * sigmoid(x).
static inline float silu_f32(float x) { return x * (std::tanh(x / 2.0f) / 2.0f + 0.5f); }
ORC_API void orc_silu_mul(const float* gate, const float* up, float* out, long long n) {
  for (long long i = 0; i < n; ++i) out[i] = silu_f32(gate[i]) * up[i];
}
ORC_API void orc_add(const float* a, const float* b, float* out, long long n) {
  for (long long i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

// composed.rs:869-967 — dense attention used by the reference's naive/full-recompute paths:
// one pass, online softmax, the accumulator round-trips through f32 `out` at every key.
// q [BH, Tq, D], k/v [B*Hkv, Tk, D(v)], window < 0 means none.
ORC_API void orc_sdpa_forward(const float* q, const float* k, const float* v, double scale, int causal,
                              long long window, float* out, long long batch, long long query_heads,
                              long long kv_heads, long long query_len, long long key_len, long long depth,
                              long long value_depth) {
  for (long long bh = 0; bh < batch * query_heads; ++bh) {
    const long long b = bh / query_heads, qh = bh % query_heads;
    const long long kv_bh = b * kv_heads + qh / (query_heads / kv_heads);
    for (long long query = 0; query < query_len; ++query) {
      const float* qrow = q + (bh * query_len + query) * depth;
      float* orow = out + (bh * query_len + query) * value_depth;
      for (long long c = 0; c < value_depth; ++c) orow[c] = 0.0f;
      double maximum = -INFINITY, denominator = 0.0;
      for (long long key = 0; key < key_len; ++key) {
        if (causal) {
          const long long end = query + (key_len > query_len ? key_len - query_len : 0);
          if (key > end) continue;
          if (window >= 0) {
            const long long lo = end + 1 > window ? end + 1 - window : 0;
            if (key < lo) continue;
          }
        }
        const float* krow = k + (kv_bh * key_len + key) * depth;
        double score = 0.0;
        for (long long d = 0; d < depth; ++d) score += (double)qrow[d] * (double)krow[d];
        score = score * scale;
        const double next_maximum = std::fmax(maximum, score);
        const double previous_scale = maximum == -INFINITY ? 0.0 : std::exp(maximum - next_maximum);
        const double weight = std::exp(score - next_maximum);
        const float* vrow = v + (kv_bh * key_len + key) * value_depth;
        for (long long c = 0; c < value_depth; ++c)
          orow[c] = (float)((double)orow[c] * previous_scale + weight * (double)vrow[c]);
        denominator = denominator * previous_scale + weight;
        maximum = next_maximum;
      }
      for (long long c = 0; c < value_depth; ++c) orow[c] = (float)((double)orow[c] / denominator);
    }
  }
}

// ----------------------------------------------------------------------------------
// Sampling (crates/runtime/src/sampling.rs).
// ----------------------------------------------------------------------------------

// sampling.rs:88-105 — greedy: first index of the maximum (strict >), in f64; a non-finite
// logit is an error. Returns the token, or -(index+1) of the first non-finite logit.
ORC_API long long orc_argmax(const float* logits, long long length) {
  long long selected = 0;
  double best = -INFINITY;
  for (long long t = 0; t < length; ++t) {
    const double value = (double)logits[t];
    if (!std::isfinite(value)) return -(t + 1);
    if (value > best) { best = value; selected = t; }
  }
  return selected;
}

static double random_unit(uint64_t seed, uint64_t counter) {  // sampling.rs:35-42
  uint64_t value = seed ^ (counter * 0x9e3779b97f4a7c15ull);
  value += 0x9e3779b97f4a7c15ull;
  value = (value ^ (value >> 30)) * 0xbf58476d1ce4e5b9ull;
  value = (value ^ (value >> 27)) * 0x94d049bb133111ebull;
  value ^= value >> 31;
  return (double)(value >> 11) * (1.0 / 9007199254740992.0);
}
ORC_API double orc_random_unit(uint64_t seed, uint64_t counter) { return random_unit(seed, counter); }

// sampling.rs:80-206 — full sampler. top_k <= 0 disables top-k. Returns token >= 0,
// -(index+1) for a non-finite logit, or -2000000000 - code for an options error
// (1 empty, 2 temperature, 3 topP, 4 topK, 5 vocabulary too large).
ORC_API long long orc_sample_logits(const float* logits, long long length, double temperature, long long top_k,
                                    double top_p, uint64_t seed, uint64_t counter) {
  const long long kOptionError = -2000000000ll;
  if (length == 0) return kOptionError - 1;
  if (length > 1048576) return kOptionError - 5;
  if (!std::isfinite(temperature) || temperature < 0.0) return kOptionError - 2;
  if (!std::isfinite(top_p) || top_p <= 0.0 || top_p > 1.0) return kOptionError - 3;
  if (top_k > 0 && top_k > length) return kOptionError - 4;
  if (temperature == 0.0) return orc_argmax(logits, length);
  const bool has_top_k = top_k > 0 && top_k < length;
  const bool filtered = has_top_k || top_p < 1.0;
  if (!filtered) {
    double max = -INFINITY;
    for (long long t = 0; t < length; ++t) {
      const double value = (double)logits[t];
      if (!std::isfinite(value)) return -(t + 1);
      max = std::fmax(max, value);
    }
    double total = 0.0;
    for (long long t = 0; t < length; ++t) total += std::exp(((double)logits[t] - max) / temperature);
    double draw = random_unit(seed, counter) * total;
    for (long long t = 0; t < length; ++t) {
      draw -= std::exp(((double)logits[t] - max) / temperature);
      if (draw < 0.0) return t;
    }
    return length - 1;
  }
  struct Candidate { long long token; double value; };
  std::vector<Candidate> candidates((size_t)length);
  for (long long t = 0; t < length; ++t) {
    const double value = (double)logits[t];
    if (!std::isfinite(value)) return -(t + 1);
    candidates[(size_t)t] = {t, value};
  }
  // Descending by value, ties to the lower token: a total order, so partial selection
  // followed by a sort (the reference) equals one full sort followed by truncation.
  std::sort(candidates.begin(), candidates.end(), [](const Candidate& l, const Candidate& r) {
    if (l.value != r.value) return l.value > r.value;
    return l.token < r.token;
  });
  if (has_top_k) candidates.resize((size_t)top_k);
  const double max = candidates[0].value;
  double total = 0.0;
  for (auto& c : candidates) {
    c.value = std::exp((c.value - max) / temperature);
    total += c.value;
  }
  size_t retained = candidates.size();
  if (top_p < 1.0) {
    const double threshold = top_p * total;
    double cumulative = 0.0;
    for (size_t i = 0; i < candidates.size(); ++i) {
      cumulative += candidates[i].value;
      if (cumulative >= threshold) {
        retained = i + 1;
        total = cumulative;
        break;
      }
    }
  }
  double draw = random_unit(seed, counter) * total;
  for (size_t i = 0; i < retained; ++i) {
    draw -= candidates[i].value;
    if (draw < 0.0) return candidates[i].token;
  }
  return candidates[retained - 1].token;
}

// crates/runtime-cpu/src/napi/mod.rs:3053-3075 — copy row advance-1 of [1,T,V] to [V].
// Returns 0, or 1 when advance is outside 1..=steps.
ORC_API int orc_last_token_row(const float* source, long long steps, long long width, long long advance, float* out) {
  if (advance <= 0 || advance > steps) return 1;
  std::memcpy(out, source + (advance - 1) * width, (size_t)width * sizeof(float));
  return 0;
}

// ----------------------------------------------------------------------------------
// KV slabs (crates/runtime-cpu/src/pool.rs).
// ----------------------------------------------------------------------------------
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_U8 = 3 };

struct Slab {  // pool.rs:32-112 — rows x row_width elements of one tier, zero-initialised
  int dtype = ORC_F32;
  size_t rows = 0, row_width = 0;
  std::vector<float> f32;
  std::vector<uint16_t> h16;
  std::vector<uint8_t> u8;
  void init(size_t r, size_t w, int dt) {
    dtype = dt; rows = r; row_width = w;
    const size_t n = r * w;
    if (dt == ORC_F32) f32.assign(n, 0.0f);
    else if (dt == ORC_U8) u8.assign(n, 0);
    else h16.assign(n, 0);
  }
  float get_f32(size_t i) const {  // pool.rs:51-58: widening read; u8 returns the raw biased code
    switch (dtype) {
      case ORC_F32: return f32[i];
      case ORC_F16: return f16_bits_to_f32(h16[i]);
      case ORC_BF16: return bf16_bits_to_f32(h16[i]);
      default: return (float)u8[i];
    }
  }
  void set_f32(size_t i, float v) {  // pool.rs:72-79: RNE narrowing on write
    switch (dtype) {
      case ORC_F32: f32[i] = v; break;
      case ORC_F16: h16[i] = f32_to_f16_bits(v); break;
      case ORC_BF16: h16[i] = f32_to_bf16_bits(v); break;
      default: std::abort();
    }
  }
};

// pool.rs:224-240 — per (row, head): scale = absmax/127 + 1e-12, code = clamp(round(x/scale),
// +-127) + 128 (round = ties away from zero).
ORC_API void orc_quantize_int8(const float* x, long long rows, long long heads, long long d, uint8_t* q, float* scales) {
  for (long long r = 0; r < rows; ++r)
    for (long long h = 0; h < heads; ++h) {
      const long long base = (r * heads + h) * d;
      float amax = 0.0f;
      for (long long j = 0; j < d; ++j) amax = std::fmax(amax, std::fabs(x[base + j]));
      const float scale = amax / 127.0f + 1e-12f;
      scales[r * heads + h] = scale;
      for (long long j = 0; j < d; ++j) {
        float v = std::round(x[base + j] / scale);
        v = v < -127.0f ? -127.0f : (v > 127.0f ? 127.0f : v);
        q[base + j] = (uint8_t)(v + 128.0f);
      }
    }
}
// pool.rs:245-257
ORC_API void orc_dequantize_int8(const uint8_t* q, const float* scales, long long rows, long long heads, long long d, float* out) {
  for (long long r = 0; r < rows; ++r)
    for (long long h = 0; h < heads; ++h)
      for (long long j = 0; j < d; ++j)
        out[(r * heads + h) * d + j] = ((float)q[(r * heads + h) * d + j] - 128.0f) * scales[r * heads + h];
}

// ----------------------------------------------------------------------------------
// Page allocator, prefix cache, sequences (napi/mod.rs:2378-2651, 3568-3622, 3632-3947).
// ----------------------------------------------------------------------------------
static const uint64_t HASH_SEED = 0xcbf29ce484222325ull;
static const uint64_t HASH_PRIME = 0x00000100000001b3ull;

// napi/mod.rs:2381-2390 — FNV-1a-64 over each token's 4 little-endian bytes, chained.
ORC_API uint64_t orc_chain_hash(uint64_t previous, const uint32_t* tokens, long long count) {
  uint64_t hash = previous;
  for (long long i = 0; i < count; ++i)
    for (int byte = 0; byte < 4; ++byte) {
      hash ^= (uint64_t)((tokens[i] >> (8 * byte)) & 0xff);
      hash *= HASH_PRIME;
    }
  return hash;
}
ORC_API uint64_t orc_hash_seed(void) { return HASH_SEED; }

struct BlockStore {  // napi/mod.rs:2444-2499
  std::vector<uint32_t> free_list;
  std::vector<uint32_t> refcounts;
  std::vector<uint8_t> has_hash;
  std::vector<uint64_t> hashes;
  std::unordered_map<uint64_t, std::vector<uint32_t>> by_hash;
  std::deque<uint32_t> lru;
  void init(size_t n) {
    free_list.resize(n);
    for (size_t i = 0; i < n; ++i) free_list[i] = (uint32_t)(n - 1 - i);  // (0..n).rev(): pop() yields 0,1,2,...
    refcounts.assign(n, 0);
    has_hash.assign(n, 0);
    hashes.assign(n, 0);
  }
  bool is_cached(uint32_t b) const {
    if (refcounts[b] != 0 || !has_hash[b]) return false;
    auto it = by_hash.find(hashes[b]);
    return it != by_hash.end() && std::find(it->second.begin(), it->second.end(), b) != it->second.end();
  }
  void uncache(uint32_t b, uint64_t hash) {
    auto it = by_hash.find(hash);
    if (it == by_hash.end()) return;
    auto& v = it->second;
    auto pos = std::find(v.begin(), v.end(), b);
    if (pos != v.end()) { *pos = v.back(); v.pop_back(); }  // swap_remove
    if (v.empty()) by_hash.erase(it);
  }
  size_t cached() const {
    size_t n = 0;
    for (auto& kv : by_hash)
      for (uint32_t b : kv.second) n += refcounts[b] == 0;
    return n;
  }
};

struct orc_pool {
  int layers, kv_heads, head_dim, block_size, max_tokens, dtype;
  std::vector<Slab> k, v, scales;  // scales[2*layer] = K scales, [2*layer+1] = V scales
  BlockStore store;
};

struct orc_seq {  // napi/mod.rs:2623-2651
  orc_pool* pool;
  std::vector<uint32_t> blocks;
  size_t head = 0, cursor = 0, advance = 0;
  uint64_t last_hash = HASH_SEED;
  std::vector<uint32_t> pending;
  bool released = false;
};

static long long pool_alloc_block(orc_pool* p) {  // napi/mod.rs:2516-2534
  BlockStore& s = p->store;
  if (!s.free_list.empty()) {
    const uint32_t b = s.free_list.back();
    s.free_list.pop_back();
    s.refcounts[b] = 1;
    s.has_hash[b] = 0;
    return b;
  }
  while (!s.lru.empty()) {
    const uint32_t candidate = s.lru.front();
    s.lru.pop_front();
    if (!s.is_cached(candidate)) continue;
    s.uncache(candidate, s.hashes[candidate]);
    s.has_hash[candidate] = 0;
    s.refcounts[candidate] = 1;
    return candidate;
  }
  return -1;
}
static long long pool_take_block(orc_pool* p, uint64_t hash) {  // :2536-2541
  auto it = p->store.by_hash.find(hash);
  if (it == p->store.by_hash.end() || it->second.empty()) return -1;
  const uint32_t b = it->second.front();
  p->store.refcounts[b] += 1;
  return b;
}
static void pool_unref_block(orc_pool* p, uint32_t b) {  // :2543-2554
  uint32_t& count = p->store.refcounts[b];
  if (count > 0) --count;
  if (count == 0) {
    if (p->store.has_hash[b]) p->store.lru.push_back(b);
    else p->store.free_list.push_back(b);
  }
}
static void pool_set_hash(orc_pool* p, uint32_t b, uint64_t hash) {  // :2556-2561
  p->store.has_hash[b] = 1;
  p->store.hashes[b] = hash;
  p->store.by_hash[hash].push_back(b);
}

// napi/mod.rs:3642-3751 — geometry rules of NativeKvPool::new (recurrent state is out of scope).
// Returns NULL and writes the reference's message into err on a geometry violation.
ORC_API orc_pool* orc_pool_create(int layers, int kv_heads, int head_dim, int max_tokens, int block_size, int dtype,
                                  char* err, int err_len) {
  auto fail = [&](const std::string& m) -> orc_pool* {
    if (err && err_len > 0) std::snprintf(err, (size_t)err_len, "%s", m.c_str());
    return nullptr;
  };
  if (dtype < ORC_F32 || dtype > ORC_U8) return fail("kv pool: dtype must be f32, f16, bf16 or u8 (int8-quantized)");
  if (layers == 0 && (kv_heads != 0 || head_dim != 0)) return fail("kv pool: heads and head dim must be zero when layers is zero");
  if (layers > 0 && (kv_heads == 0 || head_dim == 0)) return fail("kv pool: layers, kv heads and head dim must be positive");
  if (block_size <= 0 || max_tokens <= 0 || max_tokens % block_size != 0)
    return fail("kv pool: capacity " + std::to_string(max_tokens) + " must be a positive multiple of block size " +
                std::to_string(block_size));
  orc_pool* p = new orc_pool();
  p->layers = layers; p->kv_heads = kv_heads; p->head_dim = head_dim;
  p->block_size = block_size; p->max_tokens = max_tokens; p->dtype = dtype;
  p->k.resize((size_t)layers);
  p->v.resize((size_t)layers);
  if (dtype == ORC_U8) p->scales.resize((size_t)layers * 2);
  for (int l = 0; l < layers; ++l) {
    p->k[(size_t)l].init((size_t)max_tokens, (size_t)kv_heads * head_dim, dtype);
    p->v[(size_t)l].init((size_t)max_tokens, (size_t)kv_heads * head_dim, dtype);
    if (dtype == ORC_U8) {
      p->scales[(size_t)2 * l].init((size_t)max_tokens, (size_t)kv_heads, ORC_F32);
      p->scales[(size_t)2 * l + 1].init((size_t)max_tokens, (size_t)kv_heads, ORC_F32);
    }
  }
  p->store.init((size_t)(max_tokens / block_size));
  return p;
}
ORC_API void orc_pool_destroy(orc_pool* p) { delete p; }
ORC_API int orc_pool_capacity(orc_pool* p) { return p->max_tokens; }
ORC_API int orc_pool_free_blocks(orc_pool* p) { return (int)(p->store.free_list.size() + p->store.cached()); }  // :2611
ORC_API int orc_pool_cached_blocks(orc_pool* p) { return (int)p->store.cached(); }
ORC_API long long orc_pool_alloc_block(orc_pool* p) { return pool_alloc_block(p); }
ORC_API long long orc_pool_take_block(orc_pool* p, uint64_t h) { return pool_take_block(p, h); }
ORC_API void orc_pool_unref_block(orc_pool* p, uint32_t b) { pool_unref_block(p, b); }
ORC_API void orc_pool_set_hash(orc_pool* p, uint32_t b, uint64_t h) { pool_set_hash(p, b, h); }
// returns 1 and the hash when the block has one
ORC_API int orc_pool_block_hash(orc_pool* p, uint32_t b, uint64_t* h) {
  if (!p->store.has_hash[b]) return 0;
  *h = p->store.hashes[b];
  return 1;
}
ORC_API int orc_pool_refcount(orc_pool* p, uint32_t b) { return (int)p->store.refcounts[b]; }

// napi/mod.rs:1921-1980 — bytes of KV state referenced by a compiled program (recurrent terms
// passed in by the caller as extra bytes: zero for Llama-shaped models).
ORC_API long long orc_state_bytes(long long layers, long long max_tokens, long long kv_heads, long long head_dim, int dtype) {
  const long long size = dtype == ORC_F32 ? 4 : (dtype == ORC_U8 ? 1 : 2);
  long long bytes = layers * max_tokens * kv_heads * head_dim * 2 * size;
  if (dtype == ORC_U8) bytes += layers * max_tokens * kv_heads * 2 * 4;
  return bytes;
}

// Slab row helpers (pool.rs:134-219) for the slab-tier tests: layer slab, which = 0 K / 1 V.
ORC_API void orc_pool_write_rows_f32(orc_pool* p, int layer, int which, const uint32_t* rows, long long n, const float* src) {
  Slab& s = which == 0 ? p->k[(size_t)layer] : p->v[(size_t)layer];
  for (long long i = 0; i < n; ++i)
    for (size_t j = 0; j < s.row_width; ++j) s.set_f32((size_t)rows[i] * s.row_width + j, src[(size_t)i * s.row_width + j]);
}
ORC_API void orc_pool_read_rows_f32(orc_pool* p, int layer, int which, const uint32_t* rows, long long n, float* dst) {
  const Slab& s = which == 0 ? p->k[(size_t)layer] : p->v[(size_t)layer];
  for (long long i = 0; i < n; ++i)
    for (size_t j = 0; j < s.row_width; ++j) dst[(size_t)i * s.row_width + j] = s.get_f32((size_t)rows[i] * s.row_width + j);
}
// Dequantised read (u8 tier applies (code-128)*scale as napi/mod.rs:3474-3476 does).
ORC_API void orc_pool_read_rows_dequant(orc_pool* p, int layer, int which, const uint32_t* rows, long long n, float* dst) {
  const Slab& s = which == 0 ? p->k[(size_t)layer] : p->v[(size_t)layer];
  for (long long i = 0; i < n; ++i)
    for (size_t j = 0; j < s.row_width; ++j) {
      float raw = s.get_f32((size_t)rows[i] * s.row_width + j);
      if (p->dtype == ORC_U8) {
        const Slab& sc = p->scales[(size_t)2 * layer + which];
        raw = (raw - 128.0f) * sc.get_f32((size_t)rows[i] * p->kv_heads + j / (size_t)p->head_dim);
      }
      dst[(size_t)i * s.row_width + j] = raw;
    }
}

ORC_API orc_seq* orc_seq_create(orc_pool* p) {  // napi/mod.rs:3787-3819
  orc_seq* s = new orc_seq();
  s->pool = p;
  return s;
}
ORC_API void orc_seq_release(orc_seq* s) {  // :3825-3842 — idempotent; returns blocks from `head` on
  if (s->released) return;
  s->released = true;
  for (size_t i = s->head; i < s->blocks.size(); ++i) pool_unref_block(s->pool, s->blocks[i]);
  s->blocks.resize(std::min(s->head, s->blocks.size()));
  s->cursor = 0; s->advance = 0; s->last_hash = HASH_SEED; s->pending.clear();
}
ORC_API void orc_seq_destroy(orc_seq* s) { orc_seq_release(s); delete s; }
ORC_API long long orc_seq_cursor(orc_seq* s) { return (long long)s->cursor; }
ORC_API long long orc_seq_head(orc_seq* s) { return (long long)s->head; }
ORC_API uint64_t orc_seq_last_hash(orc_seq* s) { return s->last_hash; }
ORC_API long long orc_seq_num_blocks(orc_seq* s) { return (long long)s->blocks.size(); }
ORC_API void orc_seq_blocks(orc_seq* s, uint32_t* out) { std::copy(s->blocks.begin(), s->blocks.end(), out); }
ORC_API void orc_seq_set_advance(orc_seq* s, long long a) { s->advance = (size_t)a; }
ORC_API void orc_seq_set_cursor(orc_seq* s, long long c) { s->cursor = (size_t)c; }
ORC_API void orc_seq_push_block(orc_seq* s, uint32_t b) { s->blocks.push_back(b); }

// napi/mod.rs:2637-2650
ORC_API void orc_seq_note_tokens(orc_seq* s, const uint32_t* tokens, long long count) {
  orc_pool* p = s->pool;
  for (long long i = 0; i < count; ++i) {
    s->pending.push_back(tokens[i]);
    if ((int)s->pending.size() == p->block_size) {
      const uint64_t hash = orc_chain_hash(s->last_hash, s->pending.data(), (long long)s->pending.size());
      s->last_hash = hash;
      s->pending.clear();
      const size_t block_index = (s->cursor + (size_t)i) / (size_t)p->block_size;
      if (block_index < s->blocks.size()) pool_set_hash(p, s->blocks[block_index], hash);
    }
  }
}

// napi/mod.rs:3874-3946 (non-recurrent branch). Returns the matched cursor, -1 "kv sequence is
// released", -2 "prefill match: sequence already holds tokens".
ORC_API long long orc_seq_prefill_match(orc_seq* s, const uint32_t* tokens, long long count) {
  if (s->released) return -1;
  if (s->cursor > 0 || !s->blocks.empty()) return -2;
  orc_pool* p = s->pool;
  const long long matchable = (count > 0 ? count - 1 : 0) / p->block_size;
  uint64_t hash = HASH_SEED;
  for (long long i = 0; i < matchable; ++i) {
    const uint64_t next = orc_chain_hash(hash, tokens + i * p->block_size, p->block_size);
    const long long b = pool_take_block(p, next);
    if (b < 0) break;
    s->blocks.push_back((uint32_t)b);
    hash = next;
  }
  s->last_hash = hash;
  s->cursor = s->blocks.size() * (size_t)p->block_size;
  return (long long)s->cursor;
}

// napi/mod.rs:3568-3615. Returns 0 or an error code with the reference's message in err:
// 1 advance out of range, 2 "exceeds pool capacity", 3 "pool exhausted", 4 geometry mismatch.
static int kv_prepare(orc_pool* p, orc_seq* s, int layer, long long pool_window, int heads, int width, long long tokens,
                      size_t* cursor, size_t* needed, size_t* start, char* err, int err_len) {
  auto fail = [&](int code, const std::string& m) {
    if (err && err_len > 0) std::snprintf(err, (size_t)err_len, "%s", m.c_str());
    return code;
  };
  if (layer >= p->layers)
    return fail(4, "kv attention: layer " + std::to_string(layer) + " out of range for " + std::to_string(p->layers) + " pool layers");
  if (heads != p->kv_heads || width != p->head_dim)
    return fail(4, "kv attention: layer " + std::to_string(layer) + " shape [" + std::to_string(heads) + ", " +
                       std::to_string(width) + "] does not match pool geometry [" + std::to_string(p->kv_heads) + ", " +
                       std::to_string(p->head_dim) + "]");
  *cursor = s->cursor;
  const size_t advance = s->advance;
  if (advance == 0 || (long long)advance > tokens)
    return fail(1, "kv attention: advance " + std::to_string(advance) + " out of range for chunk length " + std::to_string(tokens));
  *needed = *cursor + advance;
  *start = pool_window >= 0 ? (*needed > (size_t)pool_window ? *needed - (size_t)pool_window : 0) : 0;
  if (*needed - *start > (size_t)p->max_tokens)
    return fail(2, "kv attention: live context " + std::to_string(*needed - *start) + " exceeds pool capacity " +
                       std::to_string(p->max_tokens));
  while (s->blocks.size() * (size_t)p->block_size < *needed) {
    const long long b = pool_alloc_block(p);
    if (b < 0)
      return fail(3, "kv attention: pool exhausted (" + std::to_string(p->max_tokens) + " tokens across live sequences)");
    s->blocks.push_back((uint32_t)b);
  }
  return 0;
}

// napi/mod.rs:3617-3622
ORC_API void orc_seq_evict(orc_seq* s, long long start) {
  orc_pool* p = s->pool;
  while (s->head < s->blocks.size() && (s->head + 1) * (size_t)p->block_size <= (size_t)start) {
    pool_unref_block(p, s->blocks[s->head]);
    s->head += 1;
  }
}

// napi/mod.rs:3320-3565 — scatter the chunk's new K/V rows into the layer slabs, then attend.
//   q [B,Hq,T,D], k/v [B,Hkv,T,D] f32 contiguous; out [B,Hq,T,D], zero for lanes >= active.
//   op_window  : the attention node's own window (-1 none)
//   pool_window: the schema-wide eviction window (-1 none)
//   eviction_starts[B]: SIZE_MAX initially; updated as in :3556-3560
//   mode 0 = reference-faithful (three passes, every score recomputed per output column);
//   mode 1 = identical arithmetic with each position's score/weight computed once (the cached
//            variant accumulates the same terms in the same order, so results are bit-identical);
//   threads: OpenMP threads over (lane, head) for mode 1.
// Returns 0 or the kv_prepare error code.
ORC_API int orc_kv_attention(orc_pool* p, int layer, orc_seq** seqs, long long batch, long long active, const float* q,
                             const float* k, const float* v, long long query_heads, long long kv_heads, long long tokens,
                             long long width, double scale, long long op_window, long long pool_window, float* out,
                             unsigned long long* eviction_starts, int mode, int threads, char* err, int err_len) {
  std::fill(out, out + batch * query_heads * tokens * width, 0.0f);
  const size_t bs = (size_t)p->block_size;
  for (long long b = 0; b < active; ++b) {
    orc_seq* s = seqs[b];
    size_t cursor, needed, start;
    const int rc = kv_prepare(p, s, layer, pool_window, (int)kv_heads, (int)width, tokens, &cursor, &needed, &start, err, err_len);
    if (rc) return rc;
    const size_t advance = s->advance;
    auto physical = [&](size_t position) -> size_t { return (size_t)s->blocks[position / bs] * bs + position % bs; };
    auto input_value = [&](const float* value, size_t token, size_t head, size_t column) -> float {
      return value[(((size_t)b * kv_heads + head) * tokens + token) * width + column];
    };
    Slab& ks = p->k[(size_t)layer];
    Slab& vs = p->v[(size_t)layer];
    if (p->dtype == ORC_U8) {  // :3397-3438
      for (int which = 0; which < 2; ++which) {
        const float* value = which == 0 ? k : v;
        Slab& slab = which == 0 ? ks : vs;
        Slab& sc = p->scales[(size_t)2 * layer + which];
        for (size_t token = 0; token < advance; ++token) {
          const size_t row = physical(cursor + token);
          for (size_t head = 0; head < (size_t)kv_heads; ++head) {
            float maximum = 0.0f;
            for (size_t c = 0; c < (size_t)width; ++c) maximum = std::fmax(maximum, std::fabs(input_value(value, token, head, c)));
            const float sca = maximum / 127.0f + 1e-12f;
            sc.f32[row * kv_heads + head] = sca;
            for (size_t c = 0; c < (size_t)width; ++c) {
              float code = std::round(input_value(value, token, head, c) / sca);
              code = code < -127.0f ? -127.0f : (code > 127.0f ? 127.0f : code);
              slab.u8[(row * kv_heads + head) * width + c] = (uint8_t)(code + 128.0f);
            }
          }
        }
      }
    } else {  // :3439-3459
      for (int which = 0; which < 2; ++which) {
        const float* value = which == 0 ? k : v;
        Slab& slab = which == 0 ? ks : vs;
        for (size_t token = 0; token < advance; ++token) {
          const size_t row = physical(cursor + token);
          for (size_t head = 0; head < (size_t)kv_heads; ++head)
            for (size_t c = 0; c < (size_t)width; ++c)
              slab.set_f32((row * kv_heads + head) * width + c, input_value(value, token, head, c));
        }
      }
    }
    auto cached = [&](const Slab& slab, int which, size_t position, size_t head, size_t column) -> float {  // :3466-3477
      const size_t row = physical(position);
      const float raw = slab.get_f32((row * kv_heads + head) * width + column);
      if (p->dtype != ORC_U8) return raw;
      return (raw - 128.0f) * p->scales[(size_t)2 * layer + which].f32[row * kv_heads + head];
    };
    const long long group = query_heads / kv_heads;
    if (mode == 0) {  // :3478-3540, verbatim structure
      for (long long head = 0; head < query_heads; ++head) {
        const size_t kv_head = (size_t)(head / group);
        for (long long query = 0; query < tokens; ++query) {
          const size_t end = std::min(cursor + (size_t)query + 1, needed);
          size_t begin = start;
          if (op_window >= 0) begin = std::max(end > (size_t)op_window ? end - (size_t)op_window : 0, start);
          const float* qrow = q + (((size_t)b * query_heads + head) * tokens + query) * width;
          double maximum = -INFINITY;
          for (size_t pos = begin; pos < end; ++pos) {
            double score = 0.0;
            for (size_t c = 0; c < (size_t)width; ++c) score += (double)qrow[c] * (double)cached(ks, 0, pos, kv_head, c);
            maximum = std::fmax(maximum, score * scale);
          }
          double denominator = 0.0;
          for (size_t pos = begin; pos < end; ++pos) {
            double score = 0.0;
            for (size_t c = 0; c < (size_t)width; ++c) score += (double)qrow[c] * (double)cached(ks, 0, pos, kv_head, c);
            denominator += std::exp(score * scale - maximum);
          }
          for (size_t column = 0; column < (size_t)width; ++column) {
            double result = 0.0;
            for (size_t pos = begin; pos < end; ++pos) {
              double score = 0.0;
              for (size_t d = 0; d < (size_t)width; ++d) score += (double)qrow[d] * (double)cached(ks, 0, pos, kv_head, d);
              result += std::exp(score * scale - maximum) * (double)cached(vs, 1, pos, kv_head, column);
            }
            out[(((size_t)b * query_heads + head) * tokens + query) * width + column] = (float)(result / denominator);
          }
        }
      }
    } else {
#pragma omp parallel for schedule(dynamic) num_threads(threads > 0 ? threads : 1) collapse(2)
      for (long long head = 0; head < query_heads; ++head) {
        for (long long query = 0; query < tokens; ++query) {
          const size_t kv_head = (size_t)(head / group);
          const size_t end = std::min(cursor + (size_t)query + 1, needed);
          size_t begin = start;
          if (op_window >= 0) begin = std::max(end > (size_t)op_window ? end - (size_t)op_window : 0, start);
          const float* qrow = q + (((size_t)b * query_heads + head) * tokens + query) * width;
          const size_t span = end > begin ? end - begin : 0;
          std::vector<double> weights(span);
          double maximum = -INFINITY;
          for (size_t i = 0; i < span; ++i) {
            double score = 0.0;
            for (size_t c = 0; c < (size_t)width; ++c) score += (double)qrow[c] * (double)cached(ks, 0, begin + i, kv_head, c);
            weights[i] = score * scale;
            maximum = std::fmax(maximum, weights[i]);
          }
          double denominator = 0.0;
          for (size_t i = 0; i < span; ++i) {
            weights[i] = std::exp(weights[i] - maximum);
            denominator += weights[i];
          }
          for (size_t column = 0; column < (size_t)width; ++column) {
            double result = 0.0;
            for (size_t i = 0; i < span; ++i) result += weights[i] * (double)cached(vs, 1, begin + i, kv_head, column);
            out[(((size_t)b * query_heads + head) * tokens + query) * width + column] = (float)(result / denominator);
          }
        }
      }
    }
    if (eviction_starts) {  // :3556-3560
      const unsigned long long none = ~0ull;
      eviction_starts[b] = eviction_starts[b] == none ? (unsigned long long)start
                                                      : std::max(eviction_starts[b], (unsigned long long)start);
    }
  }
  return 0;
}

// ----------------------------------------------------------------------------------
// A Llama-shaped decoder wired from the ops above, and the stateful execution transaction
// around it (napi/mod.rs:4150-4522, crates/runtime-cpu/src/executable.rs:4515-4674). The
// wiring follows packages/core/src/models/MuseGlimmer.ts:284-367 reduced to the plain
// GQA + RoPE + SwiGLU block: RMSNorm -> q,k,v linears -> RoPE(q), RoPE(k) -> KvAttention ->
// o linear -> residual add -> RMSNorm -> silu(gate) * up -> down linear -> residual add; then
// the output RMSNorm, the head linear and LastTokenRow per lane.
// ----------------------------------------------------------------------------------
struct OrcLinear {
  int codec = 0;  // 0 = dense f32 [N,K]; otherwise a block codec id with packed bytes
  const void* data = nullptr;
  long long rows = 0, columns = 0;
};

struct orc_decoder {
  int layers, d_model, q_heads, kv_heads, head_dim, ffn, vocab;
  double eps, theta;
  int rope_layout;
  long long window;  // -1 none (full causal attention on every layer)
  int batch;         // compiled batch
  OrcLinear tok_embd;  // dense f32 [V,d] or quantized
  std::vector<const float*> attn_norm, ffn_norm;
  std::vector<OrcLinear> wq, wk, wv, wo, gate, up, down;
  const float* out_norm = nullptr;
  OrcLinear head;
  int threads = 1;   // 1 = reference-faithful single thread; > 1 = fair multi-core variant
  int faithful = 1;  // 1 = re-decode per vector + D-fold recomputed attention scores
};

ORC_API orc_decoder* orc_decoder_create(int layers, int d_model, int q_heads, int kv_heads, int head_dim, int ffn, int vocab,
                                        double eps, double theta, int rope_layout, long long window, int batch) {
  orc_decoder* m = new orc_decoder();
  m->layers = layers; m->d_model = d_model; m->q_heads = q_heads; m->kv_heads = kv_heads; m->head_dim = head_dim;
  m->ffn = ffn; m->vocab = vocab; m->eps = eps; m->theta = theta; m->rope_layout = rope_layout; m->window = window;
  m->batch = batch;
  m->attn_norm.assign((size_t)layers, nullptr);
  m->ffn_norm.assign((size_t)layers, nullptr);
  m->wq.resize((size_t)layers); m->wk.resize((size_t)layers); m->wv.resize((size_t)layers); m->wo.resize((size_t)layers);
  m->gate.resize((size_t)layers); m->up.resize((size_t)layers); m->down.resize((size_t)layers);
  return m;
}
ORC_API void orc_decoder_destroy(orc_decoder* m) { delete m; }
ORC_API void orc_decoder_set_mode(orc_decoder* m, int faithful, int threads) { m->faithful = faithful; m->threads = threads; }

// which: 0 tok_embd, 1 attn_norm, 2 wq, 3 wk, 4 wv, 5 wo, 6 ffn_norm, 7 gate, 8 up, 9 down, 10 out_norm, 11 head.
// The caller keeps `data` alive. codec 0 = dense f32.
ORC_API int orc_decoder_set_weight(orc_decoder* m, int which, int layer, int codec, const void* data, long long rows, long long columns) {
  OrcLinear lin;
  lin.codec = codec; lin.data = data; lin.rows = rows; lin.columns = columns;
  const size_t l = (size_t)layer;
  switch (which) {
    case 0: m->tok_embd = lin; break;
    case 1: m->attn_norm[l] = (const float*)data; break;
    case 2: m->wq[l] = lin; break;
    case 3: m->wk[l] = lin; break;
    case 4: m->wv[l] = lin; break;
    case 5: m->wo[l] = lin; break;
    case 6: m->ffn_norm[l] = (const float*)data; break;
    case 7: m->gate[l] = lin; break;
    case 8: m->up[l] = lin; break;
    case 9: m->down[l] = lin; break;
    case 10: m->out_norm = (const float*)data; break;
    case 11: m->head = lin; break;
    default: return -1;
  }
  return 0;
}

static int run_linear(const orc_decoder* m, const OrcLinear& w, const float* x, long long vectors, float* out) {
  if (w.codec == 0) {
    orc_linear_rows_f32(x, vectors, w.columns, (const float*)w.data, w.rows, out, m->threads);
    return 0;
  }
  if (m->faithful) return orc_qlinear(w.codec, x, vectors, w.columns, (const uint8_t*)w.data, w.rows, nullptr, out, nullptr);
  return orc_qlinear_mt(w.codec, x, vectors, w.columns, (const uint8_t*)w.data, w.rows, nullptr, out, m->threads);
}

// [B,T,H*D] -> [B,H,T,D] (the reshape/transpose pair of MuseGlimmer.ts:289-298)
static void heads_first(const float* src, float* dst, long long B, long long T, long long H, long long D) {
  for (long long b = 0; b < B; ++b)
    for (long long t = 0; t < T; ++t)
      for (long long h = 0; h < H; ++h)
        std::memcpy(dst + (((b * H + h) * T + t) * D), src + (((b * T + t) * H + h) * D), (size_t)D * sizeof(float));
}
static void heads_last(const float* src, float* dst, long long B, long long T, long long H, long long D) {
  for (long long b = 0; b < B; ++b)
    for (long long h = 0; h < H; ++h)
      for (long long t = 0; t < T; ++t)
        std::memcpy(dst + (((b * T + t) * H + h) * D), src + (((b * H + h) * T + t) * D), (size_t)D * sizeof(float));
}

// One stateful invocation: `active` real sequences padded to the compiled batch with throwaway
// sequences (advance 0, token 0, cursor 0 — napi/mod.rs:4171-4176, 4422-4436); every lane
// advances by the same `advance` (:4280-4286). tokens is [active, advance] u32.
//   logits_out: [active, vocab] f32 (LastTokenRow of each active lane), may be NULL
//   sampled_out: [active] greedy tokens sampled BEFORE commit (:4467-4486), may be NULL
//   layer_limit: run only the first `layer_limit` layers (<= 0: all) — used to time a slice
// Transaction (:4441-4518, executable.rs:4593-4665): on any error the blocks allocated during
// the run are unreferenced and cursors stay put; on success tokens are noted (block hashes),
// window-dead blocks evicted, cursor += advance.
// Returns 0, a kv_prepare error code (1..4), 5 "exceeds compiled max_tokens", 6 invalid batch,
// 7 non-finite logit while sampling, 8 token id outside the vocabulary.
ORC_API int orc_decoder_execute(orc_decoder* m, orc_pool* pool, orc_seq** seqs, long long active, const uint32_t* tokens,
                                long long advance, float* logits_out, uint32_t* sampled_out, int layer_limit, char* err,
                                int err_len) {
  auto fail = [&](int code, const std::string& msg) {
    if (err && err_len > 0) std::snprintf(err, (size_t)err_len, "%s", msg.c_str());
    return code;
  };
  const long long B = m->batch, T = advance, d = m->d_model, Hq = m->q_heads, Hkv = m->kv_heads, D = m->head_dim;
  if (active <= 0 || active > B)
    return fail(6, "execute: executable accepts 1..=" + std::to_string(B) + " sequences, got " + std::to_string(active));
  if (advance <= 0) return fail(6, "kv run: expected one non-empty token list per sequence");
  for (long long i = 0; i < active; ++i) {
    if (seqs[i]->released) return fail(6, "kv sequence " + std::to_string(i) + " is released");
    if (m->window < 0 && seqs[i]->cursor + (size_t)advance > (size_t)pool->max_tokens)  // :4410-4420
      return fail(5, "execute: sequence " + std::to_string(i) + " exceeds compiled max_tokens " + std::to_string(pool->max_tokens));
  }
  std::vector<orc_seq*> lanes(seqs, seqs + active);
  std::vector<orc_seq*> padding;
  for (long long i = active; i < B; ++i) {
    padding.push_back(orc_seq_create(pool));
    lanes.push_back(padding.back());
  }
  std::vector<size_t> frontiers((size_t)B);
  std::vector<long long> cursors((size_t)B);
  for (long long i = 0; i < B; ++i) {
    lanes[(size_t)i]->advance = i < active ? (size_t)advance : 0;
    frontiers[(size_t)i] = lanes[(size_t)i]->blocks.size();
    cursors[(size_t)i] = (long long)lanes[(size_t)i]->cursor;
  }
  auto rollback = [&]() {
    for (long long i = 0; i < B; ++i) {
      orc_seq* s = lanes[(size_t)i];
      for (size_t j = frontiers[(size_t)i]; j < s->blocks.size(); ++j) pool_unref_block(pool, s->blocks[j]);
      s->blocks.resize(std::min(frontiers[(size_t)i], s->blocks.size()));
      s->advance = 0;
    }
    for (orc_seq* s : padding) orc_seq_destroy(s);
  };

  // token ids [B,T], pad lanes zero (executable.rs:3587-3622)
  std::vector<long long> ids((size_t)(B * T), 0);
  for (long long i = 0; i < active; ++i)
    for (long long t = 0; t < T; ++t) ids[(size_t)(i * T + t)] = (long long)tokens[i * T + t];
  const long long rowsBT = B * T;
  std::vector<float> hidden((size_t)(rowsBT * d)), normed((size_t)(rowsBT * d));
  if (m->tok_embd.codec == 0) {
    for (long long r = 0; r < rowsBT; ++r) {
      if (ids[(size_t)r] < 0 || ids[(size_t)r] >= m->tok_embd.rows) {
        rollback();
        return fail(8, "embedding: index " + std::to_string(ids[(size_t)r]) + " is outside 0.." + std::to_string(m->tok_embd.rows));
      }
      std::memcpy(&hidden[(size_t)(r * d)], (const float*)m->tok_embd.data + ids[(size_t)r] * d, (size_t)d * sizeof(float));
    }
  } else {
    long long bad = 0;
    if (orc_qembedding(m->tok_embd.codec, ids.data(), rowsBT, (const uint8_t*)m->tok_embd.data, m->tok_embd.rows, d,
                       hidden.data(), &bad)) {
      rollback();
      return fail(8, "quantized_embedding: index " + std::to_string(bad) + " is outside 0.." + std::to_string(m->tok_embd.rows));
    }
  }
  std::vector<float> qf((size_t)(rowsBT * Hq * D)), kf((size_t)(rowsBT * Hkv * D)), vf((size_t)(rowsBT * Hkv * D));
  std::vector<float> qh(qf.size()), kh(kf.size()), vh(vf.size()), qr(qf.size()), kr(kf.size()), att(qf.size()), attl(qf.size());
  std::vector<float> proj((size_t)(rowsBT * d)), g((size_t)(rowsBT * m->ffn)), u(g.size()), act(g.size());
  std::vector<unsigned long long> eviction_starts((size_t)B, ~0ull);
  const double scale = 1.0 / std::sqrt((double)D);
  const int nlayers = layer_limit > 0 && layer_limit < m->layers ? layer_limit : m->layers;
  for (int l = 0; l < nlayers; ++l) {
    const size_t li = (size_t)l;
    orc_rms_norm(hidden.data(), m->attn_norm[li], m->eps, normed.data(), rowsBT, d);
    run_linear(m, m->wq[li], normed.data(), rowsBT, qf.data());
    run_linear(m, m->wk[li], normed.data(), rowsBT, kf.data());
    run_linear(m, m->wv[li], normed.data(), rowsBT, vf.data());
    heads_first(qf.data(), qh.data(), B, T, Hq, D);
    heads_first(kf.data(), kh.data(), B, T, Hkv, D);
    heads_first(vf.data(), vh.data(), B, T, Hkv, D);
    // RoPE with the per-lane cursors captured at begin (napi/mod.rs:2830-2838)
    orc_rotary(qh.data(), cursors.data(), B, m->theta, 1.0, m->rope_layout, qr.data(), B, B * Hq, T, D);
    orc_rotary(kh.data(), cursors.data(), B, m->theta, 1.0, m->rope_layout, kr.data(), B, B * Hkv, T, D);
    const int rc = orc_kv_attention(pool, l, lanes.data(), B, active, qr.data(), kr.data(), vh.data(), Hq, Hkv, T, D, scale,
                                    m->window, m->window, att.data(), eviction_starts.data(), m->faithful ? 0 : 1,
                                    m->threads, err, err_len);
    if (rc) {
      rollback();
      return rc;
    }
    heads_last(att.data(), attl.data(), B, T, Hq, D);
    run_linear(m, m->wo[li], attl.data(), rowsBT, proj.data());
    orc_add(hidden.data(), proj.data(), hidden.data(), rowsBT * d);
    orc_rms_norm(hidden.data(), m->ffn_norm[li], m->eps, normed.data(), rowsBT, d);
    run_linear(m, m->gate[li], normed.data(), rowsBT, g.data());
    run_linear(m, m->up[li], normed.data(), rowsBT, u.data());
    orc_silu_mul(g.data(), u.data(), act.data(), rowsBT * m->ffn);
    run_linear(m, m->down[li], act.data(), rowsBT, proj.data());
    orc_add(hidden.data(), proj.data(), hidden.data(), rowsBT * d);
  }
  if (logits_out || sampled_out) {
    orc_rms_norm(hidden.data(), m->out_norm, m->eps, normed.data(), rowsBT, d);
    // The reference computes the head for all T rows and then selects row advance-1
    // (LastTokenRow); only that row is needed for the result, and each output element's
    // chain is independent of the others, so only the selected rows are evaluated here.
    std::vector<float> last((size_t)(active * d)), logits((size_t)(active * m->vocab));
    for (long long i = 0; i < active; ++i)
      std::memcpy(&last[(size_t)(i * d)], &normed[(size_t)((i * T + (advance - 1)) * d)], (size_t)d * sizeof(float));
    run_linear(m, m->head, last.data(), active, logits.data());
    if (logits_out) std::memcpy(logits_out, logits.data(), logits.size() * sizeof(float));
    if (sampled_out) {
      for (long long i = 0; i < active; ++i) {
        const long long tok = orc_argmax(&logits[(size_t)(i * m->vocab)], m->vocab);
        if (tok < 0) {
          rollback();
          return fail(7, "sample: logit " + std::to_string(-tok - 1) + " is not finite");
        }
        sampled_out[i] = (uint32_t)tok;
      }
    }
  }
  // commit (napi/mod.rs:2844-2877, 4511-4518)
  for (long long i = 0; i < B; ++i)
    if (eviction_starts[(size_t)i] != ~0ull) orc_seq_evict(lanes[(size_t)i], (long long)eviction_starts[(size_t)i]);
  for (long long i = 0; i < active; ++i) {
    orc_seq* s = lanes[(size_t)i];
    orc_seq_note_tokens(s, tokens + i * T, T);
    s->cursor += s->advance;
    s->advance = 0;
  }
  for (orc_seq* s : padding) orc_seq_destroy(s);
  return 0;
}

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
