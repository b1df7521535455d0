// Per-op entry points of the C ABI: validation in the style of the reference's `*_requirements`
// planners, then a launch on the runtime's stream.
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.h"
#include "kernels.h"
#include "weights.h"

using namespace etc;

namespace etc {

static etc_status check_codec_geometry(const char* operation, int codec, int64_t rows, int64_t columns, int64_t* row_bytes) {
  const int64_t rb = codec_row_bytes(codec, columns);
  if (rb < 0)
    return fail(ETC_COMPILATION, std::string(operation) + ": logical row width " + std::to_string(columns) +
                                     " is invalid for " + codec_name(codec));
  if (rows < 0 || (rb > 0 && rows > INT64_MAX / rb))
    return fail(ETC_COMPILATION, std::string(operation) + ": packed weight byte size overflow");
  if (row_bytes) *row_bytes = rb;
  return ETC_OK;
}

// The argument checks of sample_logits (crates/runtime/src/sampling.rs:44-78), same messages.
etc_status validate_sampling(int64_t length, double temperature, int64_t top_k, double top_p) {
  if (length <= 0) return fail(ETC_EXECUTION, "sample: logits must be non-empty");
  if (length > 1048576) return fail(ETC_EXECUTION, "sample: vocabulary " + std::to_string(length) + " exceeds limit 1048576");
  if (!std::isfinite(temperature) || temperature < 0.0)
    return fail(ETC_EXECUTION, "sample: temperature must be finite and non-negative, got " + std::to_string(temperature));
  if (!std::isfinite(top_p) || top_p <= 0.0 || top_p > 1.0)
    return fail(ETC_EXECUTION, "sample: topP must be finite and in (0, 1], got " + std::to_string(top_p));
  if (top_k < 0 || top_k > length)
    return fail(ETC_EXECUTION, "sample: topK must be in [1, " + std::to_string(length) + "], got " + std::to_string(top_k));
  return ETC_OK;
}

etc_status make_inv_freq(etc_runtime* rt, double theta, int head_dim, double** out_device) {
  // theta^(-2j/D) with the host pow(), as rotary_forward_into_impl evaluates it (composed.rs:2712-2716)
  const int half = head_dim / 2;
  std::vector<double> host((size_t)std::max(half, 1));
  for (int j = 0; j < half; ++j) host[(size_t)j] = std::pow(theta, -2.0 * (double)j / (double)head_dim);
  void* d = nullptr;
  ETC_TRY(rt->device_alloc(host.size() * sizeof(double), &d));
  cudaError_t e = cudaMemcpyAsync(d, host.data(), host.size() * sizeof(double), cudaMemcpyHostToDevice, rt->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
  if (e != cudaSuccess) {
    rt->device_free(d);
    return fail(ETC_TRANSFER, std::string("rope table upload failed: ") + cudaGetErrorString(e));
  }
  *out_device = (double*)d;
  return ETC_OK;
}

namespace {
bool tiled_k_quant(int codec) {
  return codec == ETC_CODEC_Q3_K || codec == ETC_CODEC_Q4_K || codec == ETC_CODEC_Q5_K || codec == ETC_CODEC_Q6_K;
}
bool tiled_nibbles(int codec) { return codec == ETC_CODEC_Q4_0 || codec == ETC_CODEC_Q4_K; }
}  // namespace

// `part_codecs` (may be null: every part is `codec`) gives each part its own codec. Parts of different codecs become
// segments: runs of 128-row tiles repacked in their own layouts, which requires every run to end on a tile boundary.
etc_status build_qweight(etc_runtime* rt, int codec, const void* const* parts, const int64_t* part_rows, int n_parts,
                         int64_t columns, int interleave8, int on_device, etc_qweight** out, const int* part_codecs) {
  if (n_parts < 1 || n_parts > 4) return fail(ETC_INVALID_ARGUMENT, "qweight: between 1 and 4 parts are supported");
  bool kquant = false, mixed = false;
  for (int p = 0; p < n_parts; ++p) {
    const int pc = part_codecs ? part_codecs[p] : codec;
    if (pc != ETC_CODEC_Q4_0 && pc != ETC_CODEC_Q8_0 && !tiled_k_quant(pc))
      return fail(ETC_UNSUPPORTED, std::string("tiled weights support Q4_0, Q8_0, Q3_K, Q4_K, Q5_K and Q6_K, got ") + codec_name(pc));
    kquant = kquant || tiled_k_quant(pc);
    mixed = mixed || pc != (part_codecs ? part_codecs[0] : codec);
  }
  if (part_codecs) codec = part_codecs[0];
  if (columns <= 0 || columns % 64 != 0 || (kquant && columns % 256 != 0))
    return fail(ETC_COMPILATION, "qweight: logical row width " + std::to_string(columns) + " must be a multiple of " + (kquant ? "256" : "64"));
  if (interleave8 && (n_parts != 2 || part_rows[0] != part_rows[1] || part_rows[0] % 8 != 0 || mixed))
    return fail(ETC_COMPILATION, "qweight: interleave8 needs two parts of equal row count divisible by 8 and of one codec");
  int64_t rows = 0;
  for (int p = 0; p < n_parts; ++p) {
    if (part_rows[p] <= 0 || !parts[p]) return fail(ETC_INVALID_ARGUMENT, "qweight: empty part");
    rows += part_rows[p];
  }
  const int64_t row_tile = 128;
  const int64_t kblocks = columns / 32;
  etc_qweight* w = new etc_qweight();
  w->rt = rt;
  TiledWeight& t = w->tiled;
  t.codec = codec;
  t.rows = rows;
  t.rows_padded = (rows + row_tile - 1) / row_tile * row_tile;
  t.columns = columns;
  t.interleave8 = interleave8;
  // Segments: runs of parts with one codec. K-quants are re-cut into 32-value blocks at load: Q4_K -> nibbles + (scale, min)
  // per block, Q5_K -> int8 codes + (scale, min) per block, Q3_K and Q6_K -> int8 codes + one scale per 16 values.
  int seg_first_part[kMaxSegments] = {0}, seg_parts[kMaxSegments] = {0};
  int n_segments = 0;
  int64_t row_cursor = 0;
  for (int p = 0; p < n_parts; ++p) {
    const int pc = part_codecs ? part_codecs[p] : codec;
    if (n_segments == 0 || t.segments[n_segments - 1].codec != pc) {
      if (row_cursor % row_tile != 0) {
        delete w;
        return fail(ETC_COMPILATION, "qweight: parts of different codecs must meet on a multiple of 128 rows, got " + std::to_string(row_cursor));
      }
      TiledSegment& seg = t.segments[n_segments];
      seg.codec = pc;
      seg.tile0 = (int)(row_cursor / row_tile);
      seg.quant_offset = t.quant_bytes;
      seg.scale_offset = t.scale_bytes;
      seg_first_part[n_segments] = p;
      ++n_segments;
    }
    TiledSegment& seg = t.segments[n_segments - 1];
    ++seg_parts[n_segments - 1];
    row_cursor += part_rows[p];
    const int64_t seg_rows_padded = (row_cursor + row_tile - 1) / row_tile * row_tile - (int64_t)seg.tile0 * row_tile;
    seg.tiles = (int)(seg_rows_padded / row_tile);
    t.quant_bytes = seg.quant_offset + (size_t)seg_rows_padded * kblocks * (tiled_nibbles(pc) ? 16 : 32);
    t.scale_bytes = seg.scale_offset + (size_t)seg_rows_padded * kblocks * (tiled_k_quant(pc) ? 4 : 2);
  }
  t.n_segments = n_segments > 1 ? n_segments : 0;
  // the small-batch matvec kernel (and its arrival tickets) serves single-codec Q4_0 / Q8_0 weights only
  const size_t counter_bytes = (kquant || mixed) ? 0 : (size_t)(t.rows_padded / 128) * sizeof(int);
  etc_status st = rt->device_alloc(t.quant_bytes, (void**)&t.quants);
  if (st == ETC_OK && t.scale_bytes) st = rt->device_alloc(t.scale_bytes, (void**)&t.scales);
  if (st == ETC_OK && counter_bytes) {
    st = rt->device_alloc(counter_bytes, (void**)&t.counters);
    if (st == ETC_OK && cudaMemsetAsync(t.counters, 0, counter_bytes, rt->stream) != cudaSuccess)
      st = fail(ETC_EXECUTION, "qweight: clearing the arrival tickets failed");
  }
  std::vector<void*> staged;
  const uint8_t* device_part[4] = {nullptr, nullptr, nullptr, nullptr};
  for (int p = 0; p < n_parts && st == ETC_OK; ++p) {
    if (on_device) {
      device_part[p] = (const uint8_t*)parts[p];
    } else {
      void* d = nullptr;
      const size_t bytes = (size_t)part_rows[p] * (size_t)codec_row_bytes(part_codecs ? part_codecs[p] : codec, columns);
      st = rt->device_alloc(bytes, &d);
      if (st != ETC_OK) break;
      staged.push_back(d);
      cudaError_t e = cudaMemcpyAsync(d, parts[p], bytes, cudaMemcpyHostToDevice, rt->stream);
      if (e != cudaSuccess) st = fail(ETC_TRANSFER, std::string("qweight upload failed: ") + cudaGetErrorString(e));
      device_part[p] = (const uint8_t*)d;
    }
  }
  for (int sgm = 0; sgm < n_segments && st == ETC_OK; ++sgm) {
    // each segment is repacked as a weight of its own: its parts, its codec, its slice of the arrays
    const TiledSegment& seg = t.segments[sgm];
    RepackParts rp;
    std::memset(&rp, 0, sizeof(rp));
    rp.n_parts = seg_parts[sgm];
    TiledWeight view;
    view.codec = seg.codec;
    view.columns = columns;
    view.interleave8 = interleave8;
    view.rows_padded = (int64_t)seg.tiles * row_tile;
    for (int q = 0; q < rp.n_parts; ++q) {
      rp.ptr[q] = device_part[seg_first_part[sgm] + q];
      rp.rows[q] = part_rows[seg_first_part[sgm] + q];
      view.rows += rp.rows[q];
    }
    view.quants = t.quants + seg.quant_offset;
    view.scales = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(t.scales) + seg.scale_offset);
    cudaError_t e = launch_repack(view, rp, rt->stream);
    rt->launches++;
    if (e != cudaSuccess) st = fail(ETC_EXECUTION, std::string("qweight repack failed: ") + cudaGetErrorString(e));
  }
  if (st == ETC_OK) {
    const cudaError_t e = cudaStreamSynchronize(rt->stream);
    if (e != cudaSuccess) st = fail(ETC_EXECUTION, std::string("qweight repack failed: ") + cudaGetErrorString(e));
  }
  const std::string message = last_error();
  for (void* d : staged) rt->device_free(d);
  if (st != ETC_OK) {
    rt->device_free(t.quants);
    rt->device_free(t.scales);
    rt->device_free(t.counters);
    delete w;
    return fail(st, message);
  }
  *out = w;
  return ETC_OK;
}

void destroy_qweight(etc_qweight* w) {
  if (!w) return;
  w->rt->device_free(w->tiled.quants);
  w->rt->device_free(w->tiled.scales);
  w->rt->device_free(w->tiled.counters);
  w->magic = 0;
  delete w;
}

}  // namespace etc

static bool valid_weight(const etc_qweight* w) { return w && w->magic == kWeightMagic; }

extern "C" {

etc_status etc_encoded_row_bytes(etc_codec codec, int64_t columns, int64_t* out_bytes) {
  int64_t rb = 0;
  ETC_TRY(check_codec_geometry("quantized", codec, 0, columns, &rb));
  *out_bytes = rb;
  return ETC_OK;
}

etc_status etc_dequantize_into(etc_runtime* rt, etc_codec codec, const void* d_packed, int64_t rows, int64_t columns,
                               float* d_out) {
  ETC_TRY(activate(rt));
  ETC_TRY(check_codec_geometry("dequantize", codec, rows, columns, nullptr));
  ETC_CUDA(launch_dequantize(codec, (const uint8_t*)d_packed, rows, columns, d_out, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_quantize_into(etc_runtime* rt, etc_codec codec, const float* d_x, int64_t rows, int64_t columns,
                             void* d_packed) {
  ETC_TRY(activate(rt));
  if (codec != ETC_CODEC_Q4_0 && codec != ETC_CODEC_Q8_0)
    return fail(ETC_UNSUPPORTED, std::string("quantize: only Q4_0 and Q8_0 are supported, got ") + codec_name(codec));
  ETC_TRY(check_codec_geometry("quantize", codec, rows, columns, nullptr));
  ETC_CUDA(launch_quantize(codec, d_x, rows, columns, (uint8_t*)d_packed, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_qlinear_requirements(etc_codec codec, int64_t vectors, int64_t rows, int64_t columns, size_t* out_bytes,
                                    size_t* scratch_bytes) {
  ETC_TRY(check_codec_geometry("quantized_linear", codec, rows, columns, nullptr));
  if (vectors < 0 || (rows > 0 && vectors > (int64_t)(SIZE_MAX / 4) / rows))
    return fail(ETC_COMPILATION, "quantized_linear: output byte size overflow");
  if (out_bytes) *out_bytes = (size_t)vectors * (size_t)rows * sizeof(float);
  if (scratch_bytes) *scratch_bytes = 0;
  return ETC_OK;
}

etc_status etc_qlinear_into(etc_runtime* rt, etc_codec codec, const float* d_x, int64_t vectors, int64_t columns,
                            const void* d_weight, int64_t rows, const float* d_bias, float* d_out,
                            const volatile int* cancelled) {
  ETC_TRY(activate(rt));
  ETC_TRY(check_codec_geometry("quantized_linear", codec, rows, columns, nullptr));
  if (cancelled && *cancelled) return fail(ETC_CANCELLED, "operation aborted");
  int launches = 0;
  ETC_CUDA(launch_qlinear_generic(codec, d_x, vectors, columns, (const uint8_t*)d_weight, rows, d_bias, d_out, rt->stream,
                                  &launches));
  rt->launches += (uint64_t)launches;
  return ETC_OK;
}

etc_status etc_qweight_create(etc_runtime* rt, etc_codec codec, const void* const* parts, const int64_t* part_rows,
                              int n_parts, int64_t columns, int interleave8, int on_device, etc_qweight** out) {
  ETC_TRY(activate(rt));
  if (!out) return fail(ETC_INVALID_ARGUMENT, "out is null");
  *out = nullptr;
  return build_qweight(rt, codec, parts, part_rows, n_parts, columns, interleave8, on_device, out);
}

etc_status etc_qweight_destroy(etc_qweight* w) {
  if (!valid_weight(w)) return fail(ETC_INVALID_HANDLE, "weight handle is invalid or destroyed");
  ETC_TRY(activate(w->rt));
  cudaStreamSynchronize(w->rt->stream);
  destroy_qweight(w);
  return ETC_OK;
}

etc_status etc_qweight_shape(const etc_qweight* w, int64_t* rows, int64_t* columns, etc_codec* codec, uint64_t* device_bytes) {
  if (!valid_weight(w)) return fail(ETC_INVALID_HANDLE, "weight handle is invalid or destroyed");
  if (rows) *rows = w->tiled.rows;
  if (columns) *columns = w->tiled.columns;
  if (codec) *codec = (etc_codec)w->tiled.codec;
  if (device_bytes) *device_bytes = w->tiled.quant_bytes + w->tiled.scale_bytes;
  return ETC_OK;
}

etc_status etc_qlinear_tiled_scratch_bytes(const etc_qweight* w, int64_t vectors, size_t* scratch_bytes) {
  if (!valid_weight(w)) return fail(ETC_INVALID_HANDLE, "weight handle is invalid or destroyed");
  *scratch_bytes = tiled_scratch_bytes(w->tiled, vectors, w->rt->sm_count);
  return ETC_OK;
}

etc_status etc_qlinear_tiled_into(etc_runtime* rt, const etc_qweight* w, const float* d_x, int64_t vectors,
                                  const float* d_bias, const float* d_residual, etc_epilogue epilogue, float* d_out,
                                  void* d_scratch, size_t scratch_bytes) {
  ETC_TRY(activate(rt));
  if (!valid_weight(w) || w->rt != rt) return fail(ETC_INVALID_HANDLE, "weight belongs to a different runtime");
  if (epilogue == ETC_EPILOGUE_SWIGLU && !w->tiled.interleave8)
    return fail(ETC_UNSUPPORTED, "quantized_linear: the swiglu epilogue needs a weight built with interleave8");
  if (epilogue == ETC_EPILOGUE_RESIDUAL && !d_residual)
    return fail(ETC_INVALID_ARGUMENT, "quantized_linear: the residual epilogue needs a residual input");
  if (vectors <= 0) return ETC_OK;
  const size_t need = tiled_scratch_bytes(w->tiled, vectors, rt->sm_count);
  void* scratch = d_scratch;
  if (need > 0) {
    if (!scratch) {
      void* ws = nullptr;
      ETC_TRY(rt->workspace(need, &ws));
      scratch = ws;
    } else if (scratch_bytes < need) {
      return fail(ETC_INVALID_ARGUMENT, "quantized_linear: scratch holds " + std::to_string(scratch_bytes) + " bytes, " +
                                            std::to_string(need) + " needed");
    }
  }
  int launches = 0;
  ETC_CUDA(launch_qlinear_tiled(w->tiled, d_x, vectors, d_bias, d_residual, epilogue, d_out, scratch, rt->d_status,
                                rt->sm_count, rt->stream, &launches));
  rt->launches += (uint64_t)launches;
  return ETC_OK;
}

etc_status etc_qembedding_into(etc_runtime* rt, etc_codec codec, const void* d_indexes, etc_index_dtype index_dtype,
                               int64_t count, const void* d_weight, int64_t rows, int64_t columns, float* d_out) {
  ETC_TRY(activate(rt));
  if (index_dtype != ETC_INDEX_U32 && index_dtype != ETC_INDEX_I64)
    return fail(ETC_UNSUPPORTED, "quantized_embedding: indexes must be u32 or i64");
  if (codec == ETC_CODEC_F32) {
    ETC_CUDA(launch_embedding_f32(d_indexes, index_dtype == ETC_INDEX_I64, count, (const float*)d_weight, rows, columns, d_out,
                                  rt->d_status, rt->stream));
  } else {
    ETC_TRY(check_codec_geometry("quantized_embedding", codec, rows, columns, nullptr));
    ETC_CUDA(launch_qembedding(codec, d_indexes, index_dtype == ETC_INDEX_I64, count, (const uint8_t*)d_weight, rows, columns,
                               d_out, rt->d_status, rt->stream));
  }
  rt->launches++;
  return ETC_OK;
}

etc_status etc_linear_f32_into(etc_runtime* rt, const float* d_x, int64_t m, int64_t k, const float* d_w, int64_t n,
                               const float* d_bias, float* d_out) {
  ETC_TRY(activate(rt));
  ETC_CUDA(launch_linear_f32(d_x, m, k, d_w, n, d_bias, d_out, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_rmsnorm_into(etc_runtime* rt, const float* d_x, const float* d_weight, double eps, int64_t rows, int64_t n,
                            float* d_out) {
  ETC_TRY(activate(rt));
  if (n <= 0) return fail(ETC_COMPILATION, "rms_norm: normalized dimension must be positive");
  ETC_CUDA(launch_rmsnorm(d_x, d_weight, eps, rows, n, d_out, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_rope_into(etc_runtime* rt, const float* d_x, const int64_t* d_offsets, int64_t n_offsets, double theta,
                         etc_rope_layout layout, int64_t batch, int64_t heads, int64_t steps, int64_t head_dim, float* d_out) {
  ETC_TRY(activate(rt));
  if (head_dim <= 0 || head_dim % 2 != 0) return fail(ETC_COMPILATION, "rotary: expected rank >= 2 and an even head dimension");
  if (n_offsets != 1 && n_offsets != batch)
    return fail(ETC_EXECUTION, "rotary embedding: " + std::to_string(n_offsets) + " offsets for batch " + std::to_string(batch));
  double* inv_freq = nullptr;
  ETC_TRY(make_inv_freq(rt, theta, (int)head_dim, &inv_freq));
  cudaError_t e = launch_rope(d_x, d_offsets, n_offsets, inv_freq, layout, batch, heads, steps, head_dim, d_out, rt->stream);
  rt->launches++;
  if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);  // the table is freed below
  rt->device_free(inv_freq);
  if (e != cudaSuccess) return fail(ETC_EXECUTION, std::string("rotary: ") + cudaGetErrorString(e));
  return ETC_OK;
}

etc_status etc_swiglu_into(etc_runtime* rt, const float* d_gate, const float* d_up, int64_t n, float* d_out) {
  ETC_TRY(activate(rt));
  ETC_CUDA(launch_swiglu(d_gate, d_up, n, d_out, 1, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_add_into(etc_runtime* rt, const float* d_a, const float* d_b, int64_t n, float* d_out) {
  ETC_TRY(activate(rt));
  ETC_CUDA(launch_add(d_a, d_b, n, d_out, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_argmax_into(etc_runtime* rt, const float* d_logits, int64_t rows, int64_t vocab, uint32_t* d_tokens) {
  ETC_TRY(activate(rt));
  if (vocab <= 0) return fail(ETC_EXECUTION, "sample: logits must be non-empty");
  if (vocab > 1048576) return fail(ETC_EXECUTION, "sample: vocabulary " + std::to_string(vocab) + " exceeds limit 1048576");
  ETC_CUDA(launch_argmax(d_logits, rows, vocab, d_tokens, rt->d_status, rt->stream));
  rt->launches++;
  return ETC_OK;
}

size_t etc_peer_region_bytes(int64_t capacity, int world) {
  return tp_region_bytes((size_t)std::max<int64_t>(capacity, 0), std::min(std::max(world, 1), kMaxTpRanks));
}

etc_status etc_peer_allreduce_into(etc_runtime* rt, int rank, int world, void* const* regions, int64_t capacity, int buffer,
                                   const float* d_partial, float* d_hidden, int64_t count, int two_shot, int64_t wait_cycles) {
  ETC_TRY(activate(rt));
  if (world < 1 || world > kMaxTpRanks || rank < 0 || rank >= world)
    return fail(ETC_INVALID_ARGUMENT, "peer all-reduce: rank " + std::to_string(rank) + " of " + std::to_string(world) + " is out of range (at most " +
                                          std::to_string(kMaxTpRanks) + " ranks)");
  if (!regions || !d_hidden || !d_partial || buffer < 0 || buffer > 1 || count < 0 || count % 4 != 0 || count > capacity)
    return fail(ETC_INVALID_ARGUMENT, "peer all-reduce: count must be a multiple of 4 within the regions' capacity, buffer 0 or 1");
  PeerView view{};
  view.rank = rank;
  view.world = world;
  for (int r = 0; r < world; ++r) {
    if (!regions[r]) return fail(ETC_INVALID_ARGUMENT, "peer all-reduce: region " + std::to_string(r) + " is null");
    tp_view_bind(view, r, static_cast<unsigned char*>(regions[r]), tp_slot_bytes((size_t)capacity), world);
  }
  if (count == 0) return ETC_OK;
  unsigned char* own = static_cast<unsigned char*>(regions[rank]);
  ETC_CUDA(launch_tp_allreduce(view, buffer, d_hidden, (size_t)count, (int)count, DeferredSum(), d_partial, two_shot != 0,
                               reinterpret_cast<uint32_t*>(own + kTpCounterOffset), wait_cycles > 0 ? wait_cycles : kTpWaitCycles,
                               rt->sm_count, rt->d_status, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_sample_rows_into(etc_runtime* rt, const float* d_logits, int64_t rows, int64_t vocab, double temperature,
                                int64_t top_k, double top_p, uint64_t seed, uint64_t counter, const uint64_t* d_seeds,
                                const uint64_t* d_counters, uint32_t* d_tokens) {
  ETC_TRY(activate(rt));
  ETC_TRY(validate_sampling(vocab, temperature, top_k, top_p));
  if (rows < 0 || !d_logits || !d_tokens) return fail(ETC_INVALID_ARGUMENT, "sample: logits and tokens must be device buffers");
  if (temperature == 0.0)
    ETC_CUDA(launch_argmax(d_logits, rows, vocab, d_tokens, rt->d_status, rt->stream));
  else
    ETC_CUDA(launch_sample_rows(d_logits, rows, vocab, temperature, top_k, top_p, seed, counter, d_seeds, d_counters, d_tokens,
                                rt->d_status, rt->stream));
  rt->launches++;
  return ETC_OK;
}

etc_status etc_sample_row(etc_runtime* rt, const float* d_logits, int64_t vocab, double temperature, int64_t top_k,
                          double top_p, uint64_t seed, uint64_t counter, uint32_t* out_token) {
  ETC_TRY(activate(rt));
  if (!out_token) return fail(ETC_INVALID_ARGUMENT, "sample: the token output is null");
  ETC_TRY(etc_sample_rows_into(rt, d_logits, 1, vocab, temperature, top_k, top_p, seed, counter, nullptr, nullptr, rt->d_sampled));
  cudaError_t e = cudaMemcpyAsync(rt->h_sampled, rt->d_sampled, sizeof(uint32_t), cudaMemcpyDeviceToHost, rt->stream);
  if (e != cudaSuccess) return fail(ETC_TRANSFER, std::string("readback failed: ") + cudaGetErrorString(e));
  ETC_TRY(rt->check_status());  // synchronises; a non-finite logit surfaces here
  *out_token = *rt->h_sampled;
  return ETC_OK;
}

}  // extern "C"
