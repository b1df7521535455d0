// Device decoders for GGUF block codecs. decode_elem<CODEC>(block, i) returns logical element i
// of one packed block with exactly the f32 operations, in the order, of the reference's
// decode_q*_k routines (crates/runtime-cpu/src/quantized.rs:117-261), so dequantised values are
// bit-identical: every multiply/subtract uses the non-contracting __fmul_rn / __fsub_rn
// intrinsics (the reference never fuses them). Q4_0 and Q8_0 follow the published 32-value block
// format: f16 scale first, then 16 nibble bytes (low nibbles = values 0..15, high nibbles =
// values 16..31, value = scale * (code - 8)) resp. 32 int8 (value = scale * code).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace etc {

enum : int { kQ4_0 = 2, kQ8_0 = 8, kQ2_K = 10, kQ3_K = 11, kQ4_K = 12, kQ5_K = 13, kQ6_K = 14 };

template <int CODEC> struct CodecTraits;
template <> struct CodecTraits<kQ4_0> { static constexpr int kValues = 32, kBytes = 18; };
template <> struct CodecTraits<kQ8_0> { static constexpr int kValues = 32, kBytes = 34; };
template <> struct CodecTraits<kQ2_K> { static constexpr int kValues = 256, kBytes = 84; };
template <> struct CodecTraits<kQ3_K> { static constexpr int kValues = 256, kBytes = 110; };
template <> struct CodecTraits<kQ4_K> { static constexpr int kValues = 256, kBytes = 144; };
template <> struct CodecTraits<kQ5_K> { static constexpr int kValues = 256, kBytes = 176; };
template <> struct CodecTraits<kQ6_K> { static constexpr int kValues = 256, kBytes = 210; };

__device__ __forceinline__ float fp16_at(const uint8_t* block, int offset) {
  const unsigned short bits = (unsigned short)(block[offset] | (block[offset + 1] << 8));
  return __half2float(__ushort_as_half(bits));
}

// quantized.rs:77-86
__device__ __forceinline__ void scale_min_k4(int index, const uint8_t* scales, int& scale, int& minimum) {
  if (index < 4) {
    scale = scales[index] & 63;
    minimum = scales[index + 4] & 63;
  } else {
    scale = (scales[index + 4] & 0x0f) | ((scales[index - 4] >> 6) << 4);
    minimum = (scales[index + 4] >> 4) | ((scales[index] >> 6) << 4);
  }
}

template <int CODEC>
__device__ __forceinline__ float decode_elem(const uint8_t* b, int i);

template <>
__device__ __forceinline__ float decode_elem<kQ4_0>(const uint8_t* b, int i) {
  const float d = fp16_at(b, 0);
  const int code = i < 16 ? (b[2 + i] & 0x0f) : (b[2 + i - 16] >> 4);
  return __fmul_rn(d, (float)(code - 8));
}

template <>
__device__ __forceinline__ float decode_elem<kQ8_0>(const uint8_t* b, int i) {
  const float d = fp16_at(b, 0);
  return __fmul_rn(d, (float)(int)(signed char)b[2 + i]);
}

// quantized.rs:117-138 — group order: half {0,1} x shift {0,2,4,6} x q_offset {0,16}
template <>
__device__ __forceinline__ float decode_elem<kQ2_K>(const uint8_t* b, int i) {
  const int group = i >> 4, within = i & 15;
  const int half = group >> 3, shift = ((group & 7) >> 1) * 2, q_offset = (group & 1) * 16;
  const float d = fp16_at(b, 80), dmin = fp16_at(b, 82);
  const int sc = b[group];
  const float dl = __fmul_rn(d, (float)(sc & 0x0f));
  const float ml = __fmul_rn(dmin, (float)(sc >> 4));
  const int q = (b[16 + half * 32 + q_offset + within] >> shift) & 3;
  return __fsub_rn(__fmul_rn(dl, (float)q), ml);
}

// quantized.rs:142-176
template <>
__device__ __forceinline__ float decode_elem<kQ3_K>(const uint8_t* b, int i) {
  const int group = i >> 4, within = i & 15;
  const int half = group >> 3, lane = (group & 7) >> 1, q_offset = (group & 1) * 16;
  const uint8_t* hmask = b;
  const uint8_t* quants = b + 32;
  const uint8_t* packed = b + 96;
  const float d = fp16_at(b, 108);
  const int low = group < 8 ? (packed[group] & 0x0f) : (packed[group - 8] >> 4);
  const int high = (packed[8 + (group & 3)] >> (2 * (group >> 2))) & 3;
  const int scale = (low | (high << 4)) - 32;
  const float dl = __fmul_rn(d, (float)scale);
  const int low_q = (quants[half * 32 + q_offset + within] >> (lane * 2)) & 3;
  const int high_q = (hmask[q_offset + within] & (1 << (half * 4 + lane))) == 0 ? 4 : 0;
  return __fmul_rn(dl, (float)(low_q - high_q));
}

// quantized.rs:180-199
template <>
__device__ __forceinline__ float decode_elem<kQ4_K>(const uint8_t* b, int i) {
  const int group = i >> 5, within = i & 31;
  const int pair = group >> 1, side = group & 1;
  const float d = fp16_at(b, 0), dmin = fp16_at(b, 2);
  int sc, mn;
  scale_min_k4(group, b + 4, sc, mn);
  const float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)mn);
  const int raw = b[16 + pair * 32 + within];
  const int code = side == 0 ? (raw & 0x0f) : (raw >> 4);
  return __fsub_rn(__fmul_rn(dl, (float)code), ml);
}

// quantized.rs:203-234
template <>
__device__ __forceinline__ float decode_elem<kQ5_K>(const uint8_t* b, int i) {
  const int group = i >> 5, within = i & 31;
  const int pair = group >> 1, side = group & 1;
  const float d = fp16_at(b, 0), dmin = fp16_at(b, 2);
  int sc, mn;
  scale_min_k4(group, b + 4, sc, mn);
  const float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)mn);
  const int raw = b[48 + pair * 32 + within];
  const int low_q = side == 0 ? (raw & 0x0f) : (raw >> 4);
  const int code = low_q + ((b[16 + within] & (1 << (pair * 2 + side))) == 0 ? 0 : 16);
  return __fsub_rn(__fmul_rn(dl, (float)code), ml);
}

// quantized.rs:238-261 — out index = half*128 + quarter*32 + index
template <>
__device__ __forceinline__ float decode_elem<kQ6_K>(const uint8_t* b, int i) {
  const int half = i >> 7, quarter = (i & 127) >> 5, index = i & 31;
  const uint8_t* ql = b + half * 64;
  const uint8_t* qh = b + 128 + half * 32;
  const float d = fp16_at(b, 208);
  const int low = (quarter & 1) ? ql[index + 32] : ql[index];
  const int low4 = (quarter & 2) ? (low >> 4) : (low & 0x0f);
  const int code = (low4 | (((qh[index] >> (2 * quarter)) & 3) << 4)) - 32;
  const int scale = (int)(signed char)b[192 + half * 8 + (index >> 4) + quarter * 2];
  return __fmul_rn(__fmul_rn(d, (float)scale), (float)code);
}

// Runtime dispatch helper: calls f.template operator()<CODEC>() for a codec id; returns false
// for an unknown id.
template <typename F>
inline bool dispatch_codec(int codec, F&& f) {
  switch (codec) {
    case kQ4_0: f.template operator()<kQ4_0>(); return true;
    case kQ8_0: f.template operator()<kQ8_0>(); return true;
    case kQ2_K: f.template operator()<kQ2_K>(); return true;
    case kQ3_K: f.template operator()<kQ3_K>(); return true;
    case kQ4_K: f.template operator()<kQ4_K>(); return true;
    case kQ5_K: f.template operator()<kQ5_K>(); return true;
    case kQ6_K: f.template operator()<kQ6_K>(); return true;
    default: return false;
  }
}

}  // namespace etc
