// Compiled decoder: the stateful executable of a Llama-shaped model behind the C ABI.
//
// Mirrors, for the CUDA backend, what `compile` + `Executable.execute/executeSampled` do on the
// reference CPU backend (crates/runtime-cpu/src/napi/mod.rs:4150-4522 and the command loop of
// crates/runtime-cpu/src/executable.rs:4515-4674): pad the active sequences to the compiled
// batch, begin a transaction (frontiers, advances, cursors), run the fixed command list, sample
// before commit, then commit (evict, note tokens, advance cursors) or roll back.
// The command list is the decode graph of a GQA + RoPE + SwiGLU block wired as
// packages/core/src/models/MuseGlimmer.ts:284-367 wires its ops.
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.h"
#include "kernels.h"
#include "pool.h"
#include "tensor_parallel.h"
#include "weights.h"

using namespace etc;

namespace {

struct BoundWeight {
  int codec = -1;          // -1 unbound; ETC_CODEC_F32 dense
  void* d_raw = nullptr;   // device copy of the raw tensor (owned)
  int64_t rows = 0, columns = 0;
  size_t bytes = 0;
};

}  // namespace

struct etc_decoder {
  uint32_t magic = kDecoderMagic;
  etc_runtime* rt = nullptr;
  etc_decoder_config cfg{};
  int max_advance = 1;
  bool finalized = false;
  bool tiled = false;  // projections run on the tensor-core tiling

  BoundWeight tok_embd, out_norm, head;
  std::vector<BoundWeight> attn_norm, ffn_norm, wq, wk, wv, wo, gate, up, down;
  std::vector<etc_qweight*> t_qkv, t_o, t_gu, t_down;
  etc_qweight* t_head = nullptr;
  double* d_inv_freq = nullptr;

  // device workspaces
  float *hidden = nullptr, *normed = nullptr, *qkv = nullptr, *qh = nullptr, *kh = nullptr, *vh = nullptr, *qr = nullptr,
        *kr = nullptr, *att = nullptr, *attl = nullptr, *proj = nullptr, *g = nullptr, *u = nullptr, *act = nullptr,
        *last = nullptr, *logits = nullptr;
  // f16 activation hand-off between kernels of the one-token fast path ([K/8][32][8] order, rows >= batch stay zero)
  __half *xh_norm = nullptr, *xh_att = nullptr, *xh_act = nullptr;
  bool xh_path = false;
  int xh_nv = 32;  // row stride of the hand-off layout: the batch padded to 32, 64 or 128
  float* lin_scratch = nullptr;
  size_t lin_scratch_bytes = 0;
  float* attn_scratch = nullptr;
  size_t attn_scratch_bytes = 0;
  double* exact_scratch = nullptr;
  size_t exact_scratch_bytes = 0;
  uint32_t* d_ids = nullptr;       // [batch * max_advance] token ids
  int64_t* d_cursors = nullptr;    // [batch] i64 cursors for RoPE
  uint32_t* d_tokens = nullptr;    // [batch] sampled tokens
  uint32_t* d_history = nullptr;   // generate_greedy: [steps][batch]
  size_t history_capacity = 0;
  int* d_step_counter = nullptr;
  LaneInfo* d_lanes = nullptr;
  int* d_tables = nullptr;
  int max_blocks = 0;
  // pinned staging
  uint32_t* h_ids = nullptr;
  int64_t* h_cursors = nullptr;
  LaneInfo* h_lanes = nullptr;
  int* h_tables = nullptr;
  uint32_t* h_tokens = nullptr;
  float* h_logits = nullptr;
  size_t h_logits_bytes = 0;
  int launches_last_step = 0;
  uint64_t weight_bytes = 0, workspace_bytes = 0;

  cudaGraphExec_t step_graph = nullptr;  // generate_greedy's one-token step
  // what the captured graph baked in: it is re-captured when any of these changes
  int graph_active = 0, graph_pages = 0, graph_ctx = 0;
  uint64_t graph_pool_uid = 0;  // the pool's serial number: a graph holds that pool's slab addresses as kernel arguments
  // execute / executeSampled with one token per sequence replay a captured step as well: the launch list only depends
  // on the number of active lanes and on an upper bound of the pages attended over (rounded up to 8 pages, so one
  // capture serves 128 steps); everything else a step reads is in device buffers the host refreshes before the launch
  cudaGraphExec_t exec_graph = nullptr;
  int exec_graph_active = 0, exec_graph_pages = 0, exec_graph_launches = 0;
  uint64_t exec_graph_pool_uid = 0;
  bool ran_eagerly = false;  // kernels configure their attributes on their first eager launch

  // tensor parallel: this decoder holds one rank's shard of every projection (rows of q/k/v/gate/up, columns of o/down)
  TpComm* tp = nullptr;
  int tp_rank = 0, tp_world = 1;
  // optional all-reduce over peer memory instead of NCCL: one exported region per rank
  // [flags 256 B][epoch + done counters 256 B][partial 0][partial 1], opened by every peer through CUDA IPC
  unsigned char* tp_region = nullptr;
  size_t tp_partial_bytes = 0;
  bool tp_two_shot = false;           // reduce-scatter + all-gather over peer memory (4 ranks and more)
  long long tp_wait_cycles = kTpWaitCycles;
  int64_t vocab_global = 0;           // > 0: the head holds rows [head_first_row, head_first_row + cfg.vocab) of this many
  int64_t head_first_row = 0;
  void* tp_peer_base[kMaxTpRanks] = {};
  PeerView tp_view{};
  bool tp_peer = false;
};

namespace {

bool valid_decoder(const etc_decoder* d) { return d && d->magic == kDecoderMagic; }

// Live blocks a lane can stage: the pool's capacity plus the blocks a windowed sequence holds between the allocation
// for a chunk and the eviction at its commit.
int decoder_max_blocks(const etc_decoder_config& c, int max_advance) {
  return c.max_tokens / c.block_size + 2 + (max_advance + c.block_size - 1) / c.block_size;
}
// Split-KV partials set aside at finalize: a captured step plans for the attended pages rounded up to 8, so the bound
// covers the longest possible table rounded up the same way.
size_t decoder_attention_reserve(const etc_decoder_config& c, int max_advance, int sm_count) {
  const int pages = (decoder_max_blocks(c, max_advance) + 7) / 8 * 8;
  return plan_attention_max_scratch(c.batch, c.q_heads, c.kv_heads, c.head_dim, pages, sm_count);
}

etc_status bind(etc_decoder* dec, BoundWeight& slot, int codec, const void* data, int64_t rows, int64_t columns, bool on_device) {
  etc_runtime* rt = dec->rt;
  size_t bytes;
  if (codec == ETC_CODEC_F32) {
    bytes = (size_t)rows * (size_t)columns * sizeof(float);
  } else {
    const int64_t rb = codec_row_bytes(codec, columns);
    if (rb < 0)
      return fail(ETC_COMPILATION, std::string("compile: logical row width ") + std::to_string(columns) + " is invalid for " +
                                       codec_name(codec));
    bytes = (size_t)rows * (size_t)rb;
  }
  if (slot.d_raw) {
    rt->device_free(slot.d_raw);
    slot.d_raw = nullptr;
  }
  ETC_TRY(rt->device_alloc(bytes, &slot.d_raw));
  cudaError_t e = cudaMemcpyAsync(slot.d_raw, data, bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, rt->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
  if (e != cudaSuccess) return fail(ETC_TRANSFER, std::string("weight upload failed: ") + cudaGetErrorString(e));
  slot.codec = codec;
  slot.rows = rows;
  slot.columns = columns;
  slot.bytes = bytes;
  return ETC_OK;
}

etc_status set_weight(etc_decoder* dec, int slot, int layer, int codec, const void* data, int64_t rows, int64_t columns,
                      bool on_device) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  ETC_TRY(activate(dec->rt));
  if (dec->finalized) return fail(ETC_COMPILATION, "compile: weights are constant once the decoder is finalized");
  const etc_decoder_config& c = dec->cfg;
  const bool per_layer = slot != ETC_W_TOK_EMBD && slot != ETC_W_OUT_NORM && slot != ETC_W_HEAD;
  if (per_layer && (layer < 0 || layer >= c.layers)) return fail(ETC_COMPILATION, "compile: layer index out of range");
  const int64_t qw = (int64_t)c.q_heads * c.head_dim, kvw = (int64_t)c.kv_heads * c.head_dim;
  int64_t er = 0, ec = 0;
  BoundWeight* target = nullptr;
  switch (slot) {
    case ETC_W_TOK_EMBD: er = dec->vocab_global > 0 ? dec->vocab_global : c.vocab; ec = c.d_model; target = &dec->tok_embd; break;
    case ETC_W_ATTN_NORM: er = 1; ec = c.d_model; target = &dec->attn_norm[(size_t)layer]; break;
    case ETC_W_Q: er = qw; ec = c.d_model; target = &dec->wq[(size_t)layer]; break;
    case ETC_W_K: er = kvw; ec = c.d_model; target = &dec->wk[(size_t)layer]; break;
    case ETC_W_V: er = kvw; ec = c.d_model; target = &dec->wv[(size_t)layer]; break;
    case ETC_W_O: er = c.d_model; ec = qw; target = &dec->wo[(size_t)layer]; break;
    case ETC_W_FFN_NORM: er = 1; ec = c.d_model; target = &dec->ffn_norm[(size_t)layer]; break;
    case ETC_W_GATE: er = c.ffn; ec = c.d_model; target = &dec->gate[(size_t)layer]; break;
    case ETC_W_UP: er = c.ffn; ec = c.d_model; target = &dec->up[(size_t)layer]; break;
    case ETC_W_DOWN: er = c.d_model; ec = c.ffn; target = &dec->down[(size_t)layer]; break;
    case ETC_W_OUT_NORM: er = 1; ec = c.d_model; target = &dec->out_norm; break;
    case ETC_W_HEAD: er = c.vocab; ec = c.d_model; target = &dec->head; break;
    default: return fail(ETC_INVALID_ARGUMENT, "compile: unknown weight slot");
  }
  if (rows != er || columns != ec)
    return fail(ETC_COMPILATION, "compile: weight slot " + std::to_string(slot) + " expects [" + std::to_string(er) + ", " +
                                     std::to_string(ec) + "], got [" + std::to_string(rows) + ", " + std::to_string(columns) + "]");
  const bool is_norm = slot == ETC_W_ATTN_NORM || slot == ETC_W_FFN_NORM || slot == ETC_W_OUT_NORM;
  if (is_norm && codec != ETC_CODEC_F32) return fail(ETC_UNSUPPORTED, "compile: norm weights must be f32");
  return bind(dec, *target, codec, data, rows, columns, on_device);
}

bool tileable(const BoundWeight& w) {
  if (w.codec == ETC_CODEC_Q3_K || w.codec == ETC_CODEC_Q4_K || w.codec == ETC_CODEC_Q5_K || w.codec == ETC_CODEC_Q6_K) return w.columns % 256 == 0;
  return (w.codec == ETC_CODEC_Q4_0 || w.codec == ETC_CODEC_Q8_0) && w.columns % 64 == 0;
}

template <typename T>
etc_status dalloc(etc_decoder* dec, T** out, size_t count) {
  void* p = nullptr;
  ETC_TRY(dec->rt->device_alloc(std::max<size_t>(count, 1) * sizeof(T), &p));
  dec->workspace_bytes += count * sizeof(T);
  *out = (T*)p;
  return ETC_OK;
}

struct StepContext {
  etc_decoder* dec;
  etc_pool* pool;
  int T;          // tokens per lane in this invocation
  int max_ctx;    // longest live context (exact attention scratch)
  int max_pages;  // most pages any lane attends over
  bool want_logits;
  int launches = 0;
};

// out = x W^T (+ epilogue) for one projection, choosing the tensor-core tiling when it exists.
etc_status run_linear(StepContext& s, const BoundWeight& raw, etc_qweight* tiled_w, const float* x, int64_t vectors, float* out,
                      int epilogue, const float* residual, const __half* xh_ready = nullptr, __half* out_xh = nullptr,
                      DeferredSum* defer = nullptr) {
  etc_decoder* d = s.dec;
  cudaStream_t stream = d->rt->stream;
  if (defer) *defer = DeferredSum();
  if (tiled_w) {
    ETC_CUDA(launch_qlinear_tiled(tiled_w->tiled, x, vectors, nullptr, residual, epilogue, out, d->lin_scratch,
                                  d->rt->d_status, d->rt->sm_count, stream, &s.launches, xh_ready, out_xh, d->xh_nv, defer));
    return ETC_OK;
  }
  float* target = epilogue == ETC_EPILOGUE_RESIDUAL ? d->proj : out;
  if (raw.codec == ETC_CODEC_F32) {
    ETC_CUDA(launch_linear_f32(x, vectors, raw.columns, (const float*)raw.d_raw, raw.rows, nullptr, target, stream));
    ++s.launches;
  } else {
    ETC_CUDA(launch_qlinear_generic(raw.codec, x, vectors, raw.columns, (const uint8_t*)raw.d_raw, raw.rows, nullptr, target,
                                    stream, &s.launches));
  }
  if (epilogue == ETC_EPILOGUE_RESIDUAL) {
    ETC_CUDA(launch_add(residual, target, vectors * raw.rows, out, stream));
    ++s.launches;
  }
  return ETC_OK;
}

// hidden += x W^T for the o and down projections. Under tensor parallelism every rank holds a column range of W and so
// a partial sum: rank 0 adds the residual, the others overwrite, and the all-reduce leaves the same hidden state on
// every rank (crates/runtime-cpu has no counterpart: the reference is single-device).
// `defer` (single device only): the projection may leave its split-K partials unsummed for the RMSNorm that follows,
// which then does hidden += sum itself.
etc_status project_into_hidden(StepContext& s, const BoundWeight& raw, etc_qweight* tiled_w, const float* x, int64_t rows,
                               const __half* xh_ready, int buffer, DeferredSum* defer = nullptr) {
  etc_decoder* d = s.dec;
  const bool sharded = d->tp_world > 1;
  if (defer) *defer = DeferredSum();
  if (sharded && d->tp_peer) {
    // the all-reduce kernel sends this rank's partial sum (added up from the projection's split-K partials on the way
    // when there are any) into the peers' regions and adds all ranks' sums onto hidden
    DeferredSum sum;
    ETC_TRY(run_linear(s, raw, tiled_w, x, rows, d->proj, ETC_EPILOGUE_NONE, nullptr, xh_ready, nullptr, &sum));
    ETC_CUDA(launch_tp_allreduce(d->tp_view, buffer, d->hidden, (size_t)rows * d->cfg.d_model, d->cfg.d_model, sum, d->proj, d->tp_two_shot,
                                 reinterpret_cast<uint32_t*>(d->tp_region + kTpCounterOffset), d->tp_wait_cycles, d->rt->sm_count,
                                 d->rt->d_status, d->rt->stream));
    ++s.launches;
    return ETC_OK;
  }
  const int epilogue = sharded && d->tp_rank != 0 ? ETC_EPILOGUE_NONE : ETC_EPILOGUE_RESIDUAL;
  ETC_TRY(run_linear(s, raw, tiled_w, x, rows, d->hidden, epilogue, epilogue == ETC_EPILOGUE_RESIDUAL ? d->hidden : nullptr, xh_ready,
                     nullptr, sharded ? nullptr : defer));
  if (sharded) {
    std::string error;
    if (!d->tp) return fail(ETC_EXECUTION, "tensor parallel: the group has neither a communicator nor attached peer regions");
    if (!tp_allreduce_sum(d->tp, d->hidden, (size_t)rows * d->cfg.d_model, d->rt->stream, &error)) return fail(ETC_EXECUTION, error);
    ++s.launches;
  }
  return ETC_OK;
}

// RMSNorm of the residual stream into the f16 hand-off layout; `pending` holds the split-K partials of the projection
// before it when that projection left them unsummed.
etc_status norm_hand_off(StepContext& s, const BoundWeight& weight, int64_t rows, DeferredSum& pending) {
  etc_decoder* d = s.dec;
  const etc_decoder_config& c = d->cfg;
  if (pending.splits > 0)
    ETC_CUDA(launch_sum_rmsnorm_xh8(d->hidden, pending, (const float*)weight.d_raw, c.rms_eps, rows, c.d_model, d->xh_norm, d->rt->stream, d->xh_nv));
  else
    ETC_CUDA(launch_rmsnorm_xh8(d->hidden, (const float*)weight.d_raw, c.rms_eps, rows, c.d_model, d->xh_norm, d->rt->stream, d->xh_nv));
  pending = DeferredSum();
  ++s.launches;
  return ETC_OK;
}

// Enqueues one invocation (all layers + head + greedy argmax) on the runtime's stream.
etc_status enqueue_step(StepContext& s) {
  etc_decoder* d = s.dec;
  const etc_decoder_config& c = d->cfg;
  cudaStream_t stream = d->rt->stream;
  const int B = c.batch, T = s.T, D = c.head_dim, Hq = c.q_heads, Hkv = c.kv_heads;
  const int64_t rows = (int64_t)B * T;
  const int64_t qw = (int64_t)Hq * D, kvw = (int64_t)Hkv * D, qkvw = qw + 2 * kvw;
  const double scale = 1.0 / std::sqrt((double)D);

  // token embedding (dense gather or block-decoded rows)
  if (d->tok_embd.codec == ETC_CODEC_F32) {
    ETC_CUDA(launch_embedding_f32(d->d_ids, 0, rows, (const float*)d->tok_embd.d_raw, d->tok_embd.rows, c.d_model, d->hidden,
                                  d->rt->d_status, stream));
  } else {
    ETC_CUDA(launch_qembedding(d->tok_embd.codec, d->d_ids, 0, rows, (const uint8_t*)d->tok_embd.d_raw, d->tok_embd.rows, c.d_model,
                               d->hidden, d->rt->d_status, stream));
  }
  ++s.launches;

  DeferredSum pending;  // partials of the last projection onto the residual stream, summed by the next RMSNorm
  for (int l = 0; l < c.layers; ++l) {
    const size_t li = (size_t)l;
    const PoolView view = s.pool->view(l);
    // one-token steps of a tiled model hand activations from kernel to kernel as f16 in the tensor-core operand order
    const bool xh = d->xh_path && T == 1;
    if (xh) {
      ETC_TRY(norm_hand_off(s, d->attn_norm[li], rows, pending));
    } else {
      ETC_CUDA(launch_rmsnorm(d->hidden, (const float*)d->attn_norm[li].d_raw, c.rms_eps, rows, c.d_model, d->normed, stream));
      ++s.launches;
    }
    const float *qp, *kp, *vp;
    int64_t stride_q, stride_kv;
    const bool fast_attention = d->tiled && !c.exact && attention_mma_supported(view, Hq, T);
    DeferredSum qkv_sum;  // the RoPE / append kernel can sum the fused projection's partials itself
    if (d->tiled) {
      ETC_TRY(run_linear(s, d->wq[li], d->t_qkv[li], d->normed, rows, d->qkv, ETC_EPILOGUE_NONE, nullptr, xh ? d->xh_norm : nullptr,
                         nullptr, fast_attention ? &qkv_sum : nullptr));
      qp = d->qkv; kp = d->qkv + qw; vp = d->qkv + qw + kvw;
      stride_q = stride_kv = qkvw;
    } else {
      float* qb = d->qkv;
      float* kb = qb + rows * qw;
      float* vb = kb + rows * kvw;
      ETC_TRY(run_linear(s, d->wq[li], nullptr, d->normed, rows, qb, ETC_EPILOGUE_NONE, nullptr));
      ETC_TRY(run_linear(s, d->wk[li], nullptr, d->normed, rows, kb, ETC_EPILOGUE_NONE, nullptr));
      ETC_TRY(run_linear(s, d->wv[li], nullptr, d->normed, rows, vb, ETC_EPILOGUE_NONE, nullptr));
      qp = qb; kp = kb; vp = vb;
      stride_q = qw; stride_kv = kvw;
    }
    if (fast_attention) {
      ETC_CUDA(launch_rope_append(view, d->qkv, d->d_lanes, d->d_tables, d->d_inv_freq, c.rope_layout, B, Hq, d->qr, stream, &qkv_sum, T));
      ++s.launches;
      const AttnPlan plan = plan_attention(B, Hq, Hkv, D, std::max(1, s.max_pages), d->rt->sm_count);
      if (plan.scratch_bytes > d->attn_scratch_bytes)
        return fail(ETC_EXECUTION, "kv attention: split plan for " + std::to_string(s.max_pages) + " pages needs " +
                                       std::to_string(plan.scratch_bytes) + " bytes of partials, the decoder holds " +
                                       std::to_string(d->attn_scratch_bytes));
      ETC_CUDA(launch_attention_mma(view, d->qr, d->d_lanes, d->d_tables, B, Hq, scale, c.window, d->attl, plan,
                                    d->attn_scratch, stream, &s.launches, xh ? d->xh_att : nullptr, d->xh_nv, T));
    } else {
      ETC_CUDA(launch_heads_first(qp, d->qh, B, T, Hq, D, stride_q, stream));
      ETC_CUDA(launch_heads_first(kp, d->kh, B, T, Hkv, D, stride_kv, stream));
      ETC_CUDA(launch_heads_first(vp, d->vh, B, T, Hkv, D, stride_kv, stream));
      ETC_CUDA(launch_rope(d->qh, d->d_cursors, B, d->d_inv_freq, c.rope_layout, B, Hq, T, D, d->qr, stream));
      ETC_CUDA(launch_rope(d->kh, d->d_cursors, B, d->d_inv_freq, c.rope_layout, B, Hkv, T, D, d->kr, stream));
      ETC_CUDA(launch_kv_append(view, d->kr, d->vh, d->d_lanes, d->d_tables, B, T, (int64_t)Hkv * T * D, (int64_t)T * D, D, stream));
      ETC_CUDA(launch_attention_exact(view, d->qr, d->d_lanes, d->d_tables, B, Hq, T, scale, c.window, d->att, d->exact_scratch,
                                      s.max_ctx, stream));
      ETC_CUDA(launch_heads_last(d->att, d->attl, B, T, Hq, D, stream));
      s.launches += 8;
    }
    const bool xh_o = xh && fast_attention;
    ETC_TRY(project_into_hidden(s, d->wo[li], d->tiled ? d->t_o[li] : nullptr, d->attl, rows, xh_o ? d->xh_att : nullptr, 0,
                                xh ? &pending : nullptr));
    if (xh) {
      ETC_TRY(norm_hand_off(s, d->ffn_norm[li], rows, pending));
    } else {
      ETC_CUDA(launch_rmsnorm(d->hidden, (const float*)d->ffn_norm[li].d_raw, c.rms_eps, rows, c.d_model, d->normed, stream));
      ++s.launches;
    }
    if (d->tiled) {
      ETC_TRY(run_linear(s, d->gate[li], d->t_gu[li], d->normed, rows, xh ? nullptr : d->act, ETC_EPILOGUE_SWIGLU, nullptr,
                         xh ? d->xh_norm : nullptr, xh ? d->xh_act : nullptr));
    } else {
      ETC_TRY(run_linear(s, d->gate[li], nullptr, d->normed, rows, d->g, ETC_EPILOGUE_NONE, nullptr));
      ETC_TRY(run_linear(s, d->up[li], nullptr, d->normed, rows, d->u, ETC_EPILOGUE_NONE, nullptr));
      ETC_CUDA(launch_swiglu(d->g, d->u, rows * c.ffn, d->act, c.exact, stream));
      ++s.launches;
    }
    ETC_TRY(project_into_hidden(s, d->down[li], d->tiled ? d->t_down[li] : nullptr, d->act, rows, xh ? d->xh_act : nullptr, 1,
                                xh ? &pending : nullptr));
  }
  const bool xh_head = d->xh_path && T == 1;
  if (xh_head) {
    ETC_TRY(norm_hand_off(s, d->out_norm, rows, pending));
  } else {
    ETC_CUDA(launch_rmsnorm(d->hidden, (const float*)d->out_norm.d_raw, c.rms_eps, rows, c.d_model, d->normed, stream));
    ++s.launches;
  }
  // LastTokenRow then the head: only the selected row of each lane reaches the head projection
  // (each head output is an independent dot product, so the result equals projecting all rows first).
  const float* head_in = d->normed;
  if (T > 1) {
    ETC_CUDA(launch_last_token_rows(d->normed, B, T, c.d_model, T, d->last, stream));
    ++s.launches;
    head_in = d->last;
  }
  ETC_TRY(run_linear(s, d->head, d->tiled ? d->t_head : nullptr, head_in, B, d->logits, ETC_EPILOGUE_NONE, nullptr,
                     xh_head ? d->xh_norm : nullptr));
  if (d->vocab_global > 0 && d->tp_world > 1) {
    // vocabulary-parallel head: every rank picks its best row, the ranks exchange (logit, token) pairs over peer memory
    if (!d->tp_peer) return fail(ETC_EXECUTION, "tensor parallel: a vocabulary-parallel head needs the peer exchange regions (etc_decoder_tp_peer_import)");
    if (B > kTpMaxPicks) return fail(ETC_UNSUPPORTED, "tensor parallel: a vocabulary-parallel head serves batches up to " + std::to_string(kTpMaxPicks));
    ETC_CUDA(launch_argmax(d->logits, B, c.vocab, d->d_tokens, d->rt->d_status, stream,
                           reinterpret_cast<uint2*>(d->tp_region + kTpPickOffset), (uint32_t)d->head_first_row));
    ETC_CUDA(launch_tp_pick(d->tp_view, B, d->d_tokens, reinterpret_cast<uint32_t*>(d->tp_region + kTpCounterOffset), d->tp_wait_cycles,
                            d->rt->d_status, stream));
    s.launches += 2;
  } else {
    ETC_CUDA(launch_argmax(d->logits, B, c.vocab, d->d_tokens, d->rt->d_status, stream));
    ++s.launches;
  }
  return ETC_OK;
}

struct Transaction {
  std::vector<etc_seq*> seqs;
  std::vector<size_t> frontiers;
  std::vector<std::unique_lock<std::mutex>> locks;
  void rollback() {
    for (size_t i = 0; i < seqs.size(); ++i) seqs[i]->rollback_to(frontiers[i]);
  }
};

// Validation + begin: locks, frontiers, page allocation, staging of lanes/tables/ids/cursors.
etc_status begin(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active, const uint32_t* h_tokens, int advance,
                 int reserve_tokens, Transaction& tx, StepContext& ctx) {
  const etc_decoder_config& c = dec->cfg;
  if (!dec->finalized) return fail(ETC_COMPILATION, "execute: the decoder is not finalized");
  if (!pool || pool->magic != kPoolMagic || pool->rt != dec->rt) return fail(ETC_INVALID_HANDLE, "kv pool belongs to a different runtime");
  if (active <= 0 || active > c.batch)  // validate_active_batch, napi/mod.rs:4056-4066
    return fail(ETC_INVALID_ARGUMENT, "execute: executable accepts 1..=" + std::to_string(c.batch) + " sequences, got " +
                                          std::to_string(active));
  if (advance <= 0) return fail(ETC_INVALID_ARGUMENT, "kv run: expected one non-empty token list per sequence");
  if (advance > dec->max_advance)
    return fail(ETC_INVALID_ARGUMENT, "execute: chunk of " + std::to_string(advance) + " tokens exceeds the compiled chunk length " +
                                          std::to_string(dec->max_advance));
  // validate_pool_schema, napi/mod.rs:4016-4035
  if (pool->max_tokens != c.max_tokens || pool->block_size != c.block_size || pool->dtype != c.kv_dtype ||
      pool->layers != c.layers || pool->kv_heads != c.kv_heads || pool->head_dim != c.head_dim)
    return fail(ETC_INVALID_ARGUMENT, "execute: pool capacity/block size/dtype/geometry does not match the compiled state schema");
  for (int i = 0; i < active; ++i) {
    etc_seq* s = seqs[i];
    if (!s || s->magic != kSeqMagic || s->pool != pool) return fail(ETC_INVALID_ARGUMENT, "kv run: batched sequences must share one pool");
    if (s->released) return fail(ETC_EXECUTION, "kv sequence " + std::to_string(i) + " is released");
    for (int j = 0; j < i; ++j)
      if (seqs[j] == s) return fail(ETC_INVALID_ARGUMENT, "kv run: duplicate sequence in batch");
  }
  // per-sequence run locks in address order (napi/mod.rs:4367-4393)
  std::vector<etc_seq*> ordered(seqs, seqs + active);
  std::sort(ordered.begin(), ordered.end());
  for (etc_seq* s : ordered) tx.locks.emplace_back(s->run_lock);
  for (int i = 0; i < active; ++i) {
    etc_seq* s = seqs[i];
    if (s->released) return fail(ETC_EXECUTION, "kv sequence " + std::to_string(i) + " is released");
    if (c.window < 0 && s->cursor + (size_t)reserve_tokens > (size_t)c.max_tokens)  // :4410-4420
      return fail(ETC_INVALID_ARGUMENT, "execute: sequence " + std::to_string(i) + " exceeds compiled max_tokens " + std::to_string(c.max_tokens));
  }
  tx.seqs.assign(seqs, seqs + active);
  tx.frontiers.resize((size_t)active);
  for (int i = 0; i < active; ++i) tx.frontiers[(size_t)i] = seqs[i]->blocks.size();

  ctx.dec = dec;
  ctx.pool = pool;
  ctx.T = advance;
  ctx.max_ctx = 1;
  ctx.max_pages = 1;
  std::memset(dec->h_lanes, 0, sizeof(LaneInfo) * (size_t)c.batch);
  std::memset(dec->h_cursors, 0, sizeof(int64_t) * (size_t)c.batch);
  std::memset(dec->h_ids, 0, sizeof(uint32_t) * (size_t)c.batch * (size_t)advance);  // pad lanes feed token 0
  for (int i = 0; i < active; ++i) {
    etc_seq* s = seqs[i];
    s->advance = (size_t)reserve_tokens;
    size_t cursor, needed, start;
    etc_status st = kv_prepare(pool, s, 0, c.window, c.kv_heads, c.head_dim, std::max(reserve_tokens, advance), &cursor, &needed, &start);
    if (st != ETC_OK) {
      const std::string message = last_error();
      tx.rollback();
      return fail(st, message);
    }
    s->advance = (size_t)advance;
    LaneInfo& info = dec->h_lanes[i];
    info.cursor = (int)cursor;
    info.advance = advance;
    const size_t step_needed = cursor + (size_t)advance;
    info.start = c.window >= 0 ? (int)(step_needed > (size_t)c.window ? step_needed - (size_t)c.window : 0) : 0;
    // Only live blocks [head, size) are staged; the offset is rebased so that table[pos / block_size] still
    // indexes by absolute position (a windowed sequence keeps an unbounded cursor while its live table is short).
    const size_t live = s->blocks.size() - std::min(s->head, s->blocks.size());
    if ((int)live > dec->max_blocks) {
      tx.rollback();
      return fail(ETC_EXECUTION, "execute: block table exceeds the compiled capacity");
    }
    info.table_offset = i * dec->max_blocks - (int)s->head;
    for (size_t b = 0; b < live; ++b) dec->h_tables[(size_t)i * dec->max_blocks + b] = (int)s->blocks[s->head + b];
    dec->h_cursors[i] = (int64_t)cursor;
    ctx.max_ctx = std::max(ctx.max_ctx, (int)(needed - start));
    const int first_page = info.start / c.block_size;
    ctx.max_pages = std::max(ctx.max_pages, (int)((needed + c.block_size - 1) / c.block_size) - first_page);
    for (int t = 0; t < advance; ++t) dec->h_ids[(size_t)i * advance + t] = h_tokens[(size_t)i * advance + t];
  }
  return ETC_OK;
}

etc_status upload_step_inputs(etc_decoder* dec, int advance) {
  const etc_decoder_config& c = dec->cfg;
  cudaStream_t stream = dec->rt->stream;
  ETC_CUDA(cudaMemcpyAsync(dec->d_lanes, dec->h_lanes, sizeof(LaneInfo) * (size_t)c.batch, cudaMemcpyHostToDevice, stream));
  ETC_CUDA(cudaMemcpyAsync(dec->d_tables, dec->h_tables, sizeof(int) * (size_t)c.batch * dec->max_blocks, cudaMemcpyHostToDevice, stream));
  ETC_CUDA(cudaMemcpyAsync(dec->d_cursors, dec->h_cursors, sizeof(int64_t) * (size_t)c.batch, cudaMemcpyHostToDevice, stream));
  ETC_CUDA(cudaMemcpyAsync(dec->d_ids, dec->h_ids, sizeof(uint32_t) * (size_t)c.batch * advance, cudaMemcpyHostToDevice, stream));
  return ETC_OK;
}

etc_status ensure_exact_scratch(etc_decoder* dec, const StepContext& ctx) {
  const etc_decoder_config& c = dec->cfg;
  const size_t need = (size_t)c.batch * c.q_heads * ctx.T * (size_t)ctx.max_ctx * sizeof(double);
  if (need <= dec->exact_scratch_bytes) return ETC_OK;
  ETC_CUDA(cudaStreamSynchronize(dec->rt->stream));
  if (dec->exact_scratch) dec->rt->device_free(dec->exact_scratch);
  dec->exact_scratch = nullptr;
  dec->exact_scratch_bytes = 0;
  void* p = nullptr;
  ETC_TRY(dec->rt->device_alloc(need * 2, &p));
  dec->exact_scratch = (double*)p;
  dec->exact_scratch_bytes = need * 2;
  return ETC_OK;
}

bool uses_exact_attention(const etc_decoder* dec, const etc_pool* pool, int T) {
  return !(dec->tiled && !dec->cfg.exact && attention_mma_supported(pool->view(0), dec->cfg.q_heads, T));
}

etc_status execute_impl(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active, const uint32_t* h_tokens, int advance,
                        float* h_logits, uint32_t* h_out_tokens, const volatile int* cancelled) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  etc_runtime* rt = dec->rt;
  ETC_TRY(activate(rt));
  if (!h_tokens) return fail(ETC_INVALID_ARGUMENT, "kv run: expected one non-empty token list per sequence");
  if (cancelled && *cancelled) return fail(ETC_CANCELLED, "operation aborted");
  Transaction tx;
  StepContext ctx{};
  ETC_TRY(begin(dec, pool, seqs, active, h_tokens, advance, advance, tx, ctx));
  auto abort_with = [&](etc_status st) {
    const std::string message = last_error();
    cudaStreamSynchronize(rt->stream);
    tx.rollback();
    return fail(st, message);
  };
  if (uses_exact_attention(dec, pool, advance)) {
    etc_status st = ensure_exact_scratch(dec, ctx);
    if (st != ETC_OK) return abort_with(st);
  }
  etc_status st = upload_step_inputs(dec, advance);
  if (st != ETC_OK) return abort_with(st);
  if (advance == 1 && dec->ran_eagerly && !uses_exact_attention(dec, pool, 1)) {
    const int bucket = (ctx.max_pages + 7) / 8 * 8;
    if (dec->exec_graph && (dec->exec_graph_active != active || dec->exec_graph_pages != bucket || dec->exec_graph_pool_uid != pool->uid)) {
      cudaGraphExecDestroy(dec->exec_graph);
      dec->exec_graph = nullptr;
    }
    if (!dec->exec_graph) {
      StepContext sc = ctx;
      sc.launches = 0;
      sc.max_pages = bucket;
      cudaGraph_t graph = nullptr;
      cudaError_t ce = cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeThreadLocal);
      if (ce == cudaSuccess) {
        st = enqueue_step(sc);
        const cudaError_t ce2 = cudaStreamEndCapture(rt->stream, &graph);
        if (st == ETC_OK && ce2 != cudaSuccess) ce = ce2;
      }
      if (st == ETC_OK && ce == cudaSuccess) ce = cudaGraphInstantiate(&dec->exec_graph, graph, 0);
      if (graph) cudaGraphDestroy(graph);
      if (st != ETC_OK) return abort_with(st);
      if (ce != cudaSuccess) {
        fail(ETC_EXECUTION, std::string("kv run: graph capture failed: ") + cudaGetErrorString(ce));
        return abort_with(ETC_EXECUTION);
      }
      dec->exec_graph_active = active;
      dec->exec_graph_pages = bucket;
      dec->exec_graph_pool_uid = pool->uid;
      dec->exec_graph_launches = sc.launches;
    }
    const cudaError_t ce = cudaGraphLaunch(dec->exec_graph, rt->stream);
    if (ce != cudaSuccess) {
      fail(ETC_EXECUTION, std::string("kv run: graph launch failed: ") + cudaGetErrorString(ce));
      return abort_with(ETC_EXECUTION);
    }
    ctx.launches = dec->exec_graph_launches;
  } else {
    st = enqueue_step(ctx);
    if (st != ETC_OK) return abort_with(st);
    if (advance == 1) dec->ran_eagerly = true;
  }
  dec->launches_last_step = ctx.launches;
  rt->launches += (uint64_t)ctx.launches;
  const etc_decoder_config& c = dec->cfg;
  cudaError_t e = cudaSuccess;
  if (h_out_tokens) e = cudaMemcpyAsync(dec->h_tokens, dec->d_tokens, sizeof(uint32_t) * (size_t)c.batch, cudaMemcpyDeviceToHost, rt->stream);
  if (e == cudaSuccess && h_logits)
    e = cudaMemcpyAsync(dec->h_logits, dec->logits, sizeof(float) * (size_t)active * c.vocab, cudaMemcpyDeviceToHost, rt->stream);
  if (e != cudaSuccess) {
    fail(ETC_TRANSFER, std::string("readback failed: ") + cudaGetErrorString(e));
    return abort_with(ETC_TRANSFER);
  }
  // sample-before-commit: the status word carries embedding / non-finite-logit problems
  st = rt->check_status();
  if (st != ETC_OK) {
    // a non-finite logit only matters when sampling was requested (execute() publishes logits as they are)
    const bool sampling_error = last_error().rfind("sample:", 0) == 0;
    if (!(sampling_error && !h_out_tokens)) return abort_with(st);
  }
  // cancel vs commit: one winner (crates/napi/src/lib.rs:56-82) — the flag is read once here
  if (cancelled && *cancelled) {
    fail(ETC_CANCELLED, "operation aborted");
    return abort_with(ETC_CANCELLED);
  }
  if (h_out_tokens) std::memcpy(h_out_tokens, dec->h_tokens, sizeof(uint32_t) * (size_t)active);
  if (h_logits) std::memcpy(h_logits, dec->h_logits, sizeof(float) * (size_t)active * c.vocab);
  for (int i = 0; i < active; ++i) {
    etc_seq* s = seqs[i];
    const int start = dec->h_lanes[i].start;
    if (c.window >= 0) s->evict((size_t)start);
    s->note_tokens(h_tokens + (size_t)i * advance, (size_t)advance);
    s->cursor += (size_t)advance;
    s->advance = 0;
  }
  return ETC_OK;
}

// record of one greedy step, run as the last node of the captured step graph
}  // namespace


extern "C" {

etc_status etc_kv_attention_plan(int batch, int q_heads, int kv_heads, int head_dim, int attended_pages, int sm_count,
                                 int* splits, int* pages_per_split, size_t* partial_bytes) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || attended_pages <= 0 || sm_count <= 0)
    return fail(ETC_INVALID_ARGUMENT, "kv attention plan: every argument must be positive");
  const AttnPlan p = plan_attention(batch, q_heads, kv_heads, head_dim, attended_pages, sm_count);
  if (splits) *splits = p.splits;
  if (pages_per_split) *pages_per_split = p.pages_per_split;
  if (partial_bytes) *partial_bytes = p.scratch_bytes;
  return ETC_OK;
}

etc_status etc_decoder_attention_reserve(const etc_decoder_config* config, int max_advance, int sm_count, int* max_blocks,
                                         size_t* partial_bytes) {
  if (!config || max_advance <= 0 || sm_count <= 0 || config->block_size <= 0 || config->max_tokens <= 0 || config->batch <= 0 ||
      config->q_heads <= 0 || config->kv_heads <= 0 || config->head_dim <= 0)
    return fail(ETC_INVALID_ARGUMENT, "decoder attention reserve: configuration, chunk length and SM count must be positive");
  if (max_blocks) *max_blocks = decoder_max_blocks(*config, max_advance);
  if (partial_bytes) *partial_bytes = decoder_attention_reserve(*config, max_advance, sm_count);
  return ETC_OK;
}

etc_status etc_decoder_create(etc_runtime* rt, const etc_decoder_config* config, etc_decoder** out) {
  ETC_TRY(activate(rt));
  if (!config || !out) return fail(ETC_INVALID_ARGUMENT, "compile: config and out must not be null");
  *out = nullptr;
  const etc_decoder_config& c = *config;
  if (c.layers <= 0 || c.d_model <= 0 || c.q_heads <= 0 || c.kv_heads <= 0 || c.head_dim <= 0 || c.ffn <= 0 || c.vocab <= 0)
    return fail(ETC_COMPILATION, "compile: decoder geometry must be positive");
  if (c.q_heads % c.kv_heads != 0) return fail(ETC_COMPILATION, "compile: incompatible grouped-query q/k/v shapes");
  if (c.head_dim % 2 != 0) return fail(ETC_COMPILATION, "rotary: expected rank >= 2 and an even head dimension");
  if (c.max_tokens <= 0 || c.block_size <= 0 || c.max_tokens % c.block_size != 0)  // KvStateSchema::from_native
    return fail(ETC_COMPILATION, "compile: KV max_tokens must be positive and divisible by block_size");
  if (c.batch <= 0) return fail(ETC_COMPILATION, "compile: KV batch must be positive");
  if (c.kv_dtype < ETC_KV_F32 || c.kv_dtype > ETC_KV_U8) return fail(ETC_COMPILATION, "compile: unsupported KV state dtype");
  if (c.window != ETC_NO_WINDOW && (c.window <= 0 || c.window > c.max_tokens))
    return fail(ETC_COMPILATION, "compile: KV window must be in 1..=max_tokens");
  etc_decoder* d = new etc_decoder();
  d->rt = rt;
  d->cfg = c;
  const size_t L = (size_t)c.layers;
  d->attn_norm.resize(L); d->ffn_norm.resize(L); d->wq.resize(L); d->wk.resize(L); d->wv.resize(L); d->wo.resize(L);
  d->gate.resize(L); d->up.resize(L); d->down.resize(L);
  *out = d;
  return ETC_OK;
}

etc_status etc_decoder_set_weight(etc_decoder* dec, etc_weight_slot slot, int layer, etc_codec codec, const void* h_data,
                                  int64_t rows, int64_t columns) {
  return set_weight(dec, slot, layer, codec, h_data, rows, columns, false);
}
etc_status etc_decoder_set_weight_device(etc_decoder* dec, etc_weight_slot slot, int layer, etc_codec codec, const void* d_data,
                                         int64_t rows, int64_t columns) {
  return set_weight(dec, slot, layer, codec, d_data, rows, columns, true);
}

etc_status etc_decoder_set_max_advance(etc_decoder* dec, int max_advance) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  if (dec->finalized) return fail(ETC_COMPILATION, "compile: the chunk length is fixed once the decoder is finalized");
  if (max_advance <= 0) return fail(ETC_COMPILATION, "compile: chunk length must be positive");
  dec->max_advance = max_advance;
  return ETC_OK;
}

etc_status etc_decoder_set_head_shard(etc_decoder* dec, int64_t vocab_global, int64_t first_row) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  if (dec->finalized || dec->tok_embd.d_raw || dec->head.d_raw)
    return fail(ETC_COMPILATION, "compile: the head shard is fixed before the embedding and the head are bound");
  if (vocab_global <= 0 || first_row < 0 || first_row + dec->cfg.vocab > vocab_global || vocab_global > 0xffffffffll)
    return fail(ETC_COMPILATION, "compile: head rows [" + std::to_string(first_row) + ", " + std::to_string(first_row + dec->cfg.vocab) +
                                     ") do not lie inside a vocabulary of " + std::to_string(vocab_global));
  dec->vocab_global = vocab_global;
  dec->head_first_row = first_row;
  return ETC_OK;
}

etc_status etc_tp_unique_id(uint8_t* out_id) {
  if (!out_id) return fail(ETC_INVALID_ARGUMENT, "tensor parallel: the id buffer is null");
  std::string error;
  if (!tp_unique_id(out_id, &error)) return fail(ETC_UNAVAILABLE, "tensor parallel: " + error);
  return ETC_OK;
}

etc_status etc_decoder_set_tensor_parallel(etc_decoder* dec, int rank, int world, const uint8_t* id) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  if (world < 1 || rank < 0 || rank >= world) return fail(ETC_INVALID_ARGUMENT, "tensor parallel: rank " + std::to_string(rank) + " is outside 0.." + std::to_string(world));
  if (dec->tp) return fail(ETC_COMPILATION, "tensor parallel: the decoder already has a communicator");
  if (world == 1) return ETC_OK;
  if (dec->tp_world > 1) return fail(ETC_COMPILATION, "tensor parallel: the decoder already belongs to a group");
  ETC_TRY(activate(dec->rt));
  if (id) {  // without an id there is no NCCL communicator: the ranks exchange through peer regions only
    std::string error;
    dec->tp = tp_comm_create(rank, world, id, &error);
    if (!dec->tp) return fail(ETC_UNAVAILABLE, "tensor parallel: " + error);
  }
  dec->tp_rank = rank;
  dec->tp_world = world;
  if (dec->step_graph) {  // captured without the all-reduces
    cudaGraphExecDestroy(dec->step_graph);
    dec->step_graph = nullptr;
  }
  if (dec->exec_graph) {
    cudaGraphExecDestroy(dec->exec_graph);
    dec->exec_graph = nullptr;
  }
  return ETC_OK;
}

namespace {

etc_status ensure_tp_region(etc_decoder* dec) {
  if (!dec->finalized) return fail(ETC_COMPILATION, "tensor parallel: finalize the decoder before exporting its exchange region");
  if (dec->tp_world < 2 || dec->tp_world > kMaxTpRanks)
    return fail(ETC_UNSUPPORTED, "tensor parallel: the peer-memory all-reduce serves 2 to " + std::to_string(kMaxTpRanks) + " ranks");
  etc_runtime* rt = dec->rt;
  ETC_TRY(activate(rt));
  if (!dec->tp_region) {
    const size_t floats = (size_t)dec->cfg.batch * dec->max_advance * dec->cfg.d_model;
    dec->tp_partial_bytes = tp_slot_bytes(floats);
    const size_t bytes = tp_region_bytes(floats, dec->tp_world);
    ETC_TRY(rt->device_alloc(bytes, (void**)&dec->tp_region));
    ETC_CUDA(cudaMemsetAsync(dec->tp_region, 0, bytes, rt->stream));
    ETC_CUDA(cudaStreamSynchronize(rt->stream));  // peers may write flags as soon as they hold the handle
  }
  return ETC_OK;
}

// regions[r]: rank r's region as mapped in this process (own slot: the decoder's own region)
etc_status bind_peers(etc_decoder* dec, unsigned char* const* regions) {
  PeerView view{};
  view.rank = dec->tp_rank;
  view.world = dec->tp_world;
  for (int r = 0; r < dec->tp_world; ++r) tp_view_bind(view, r, regions[r], dec->tp_partial_bytes, dec->tp_world);
  dec->tp_view = view;
  dec->tp_peer = true;
  // measured at 4 ranks, 2 MB messages: one shot 17.1 ms per step, two shot 18.2 (the second flag exchange costs more than the
  // 3 MB of extra stores); at 8 ranks one shot would send 14 MB per rank and all-reduce
  dec->tp_two_shot = dec->tp_world >= 8;
  if (const char* forced = std::getenv("ETC_TP_TWO_SHOT")) dec->tp_two_shot = std::atoi(forced) != 0;
  if (dec->step_graph) {  // captured with the NCCL all-reduces
    cudaGraphExecDestroy(dec->step_graph);
    dec->step_graph = nullptr;
  }
  if (dec->exec_graph) {
    cudaGraphExecDestroy(dec->exec_graph);
    dec->exec_graph = nullptr;
  }
  return ETC_OK;
}

}  // namespace

etc_status etc_decoder_tp_peer_export(etc_decoder* dec, uint8_t* out_handle) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  if (!out_handle) return fail(ETC_INVALID_ARGUMENT, "tensor parallel: the handle buffer is null");
  ETC_TRY(ensure_tp_region(dec));
  cudaIpcMemHandle_t handle;
  ETC_CUDA(cudaIpcGetMemHandle(&handle, dec->tp_region));
  static_assert(sizeof(handle) == 64, "CUDA IPC handles are 64 bytes");
  std::memcpy(out_handle, &handle, sizeof(handle));
  return ETC_OK;
}

etc_status etc_decoder_tp_peer_import(etc_decoder* dec, const uint8_t* handles) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  if (!handles) return fail(ETC_INVALID_ARGUMENT, "tensor parallel: the handle table is null");
  if (!dec->tp_region) return fail(ETC_COMPILATION, "tensor parallel: export this rank's region before importing the peers'");
  if (dec->tp_peer) return fail(ETC_COMPILATION, "tensor parallel: the peers are already mapped");
  etc_runtime* rt = dec->rt;
  ETC_TRY(activate(rt));
  unsigned char* regions[kMaxTpRanks] = {};
  for (int r = 0; r < dec->tp_world; ++r) {
    regions[r] = dec->tp_region;
    if (r != dec->tp_rank) {
      cudaIpcMemHandle_t handle;
      std::memcpy(&handle, handles + (size_t)r * 64, sizeof(handle));
      void* mapped = nullptr;
      ETC_CUDA(cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess));
      dec->tp_peer_base[r] = mapped;
      regions[r] = static_cast<unsigned char*>(mapped);
    }
  }
  return bind_peers(dec, regions);
}

etc_status etc_decoder_tp_region(etc_decoder* dec, void** out_region, size_t* out_bytes) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  ETC_TRY(ensure_tp_region(dec));
  if (out_region) *out_region = dec->tp_region;
  if (out_bytes) *out_bytes = tp_region_bytes((size_t)dec->cfg.batch * dec->max_advance * dec->cfg.d_model, dec->tp_world);
  return ETC_OK;
}

etc_status etc_decoder_tp_peer_attach(etc_decoder* dec, void* const* peer_regions) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  if (!peer_regions) return fail(ETC_INVALID_ARGUMENT, "tensor parallel: the region table is null");
  if (dec->tp_peer) return fail(ETC_COMPILATION, "tensor parallel: the peers are already mapped");
  ETC_TRY(ensure_tp_region(dec));
  unsigned char* regions[kMaxTpRanks] = {};
  for (int r = 0; r < dec->tp_world; ++r) {
    regions[r] = r == dec->tp_rank ? dec->tp_region : static_cast<unsigned char*>(peer_regions[r]);
    if (!regions[r]) return fail(ETC_INVALID_ARGUMENT, "tensor parallel: the region of rank " + std::to_string(r) + " is null");
  }
  return bind_peers(dec, regions);
}

etc_status etc_decoder_set_wait_limit(etc_decoder* dec, int64_t cycles) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  dec->tp_wait_cycles = cycles > 0 ? cycles : kTpWaitCycles;
  if (dec->step_graph) {  // the limit is a kernel argument of the captured all-reduces
    cudaGraphExecDestroy(dec->step_graph);
    dec->step_graph = nullptr;
  }
  if (dec->exec_graph) {
    cudaGraphExecDestroy(dec->exec_graph);
    dec->exec_graph = nullptr;
  }
  return ETC_OK;
}

etc_status etc_decoder_finalize(etc_decoder* dec) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  etc_runtime* rt = dec->rt;
  ETC_TRY(activate(rt));
  if (dec->finalized) return ETC_OK;
  const etc_decoder_config& c = dec->cfg;
  const size_t L = (size_t)c.layers;
  auto bound = [](const BoundWeight& w) { return w.codec >= 0 && w.d_raw; };
  bool all = bound(dec->tok_embd) && bound(dec->out_norm) && bound(dec->head);
  for (size_t l = 0; l < L && all; ++l)
    all = bound(dec->attn_norm[l]) && bound(dec->ffn_norm[l]) && bound(dec->wq[l]) && bound(dec->wk[l]) && bound(dec->wv[l]) &&
          bound(dec->wo[l]) && bound(dec->gate[l]) && bound(dec->up[l]) && bound(dec->down[l]);
  if (!all) return fail(ETC_COMPILATION, "compile: every weight slot of every layer must be bound before finalize");

  // Tensor-core tiling when every projection has a tiled form (Q4_0, Q8_0, Q3_K - Q6_K) and exact order was not requested.
  bool tiled = !c.exact && tileable(dec->head) && c.ffn % 8 == 0;
  // q, k and v may differ in codec (GGUF files keep v, and only v, at more bits in some layers): the fused weight then
  // holds one segment per run of equal codecs, which must meet on a 128-row tile boundary
  auto qkv_fusable = [&](size_t l) {
    const BoundWeight &q = dec->wq[l], &k = dec->wk[l], &v = dec->wv[l];
    if (!tileable(q) || !tileable(k) || !tileable(v)) return false;
    if (k.codec != q.codec && q.rows % 128 != 0) return false;
    if (v.codec != k.codec && (q.rows + k.rows) % 128 != 0) return false;
    return true;
  };
  for (size_t l = 0; l < L && tiled; ++l)
    tiled = qkv_fusable(l) && tileable(dec->wo[l]) && tileable(dec->gate[l]) && dec->up[l].codec == dec->gate[l].codec &&
            tileable(dec->down[l]);
  dec->tiled = tiled;
  auto release_raw = [&](BoundWeight& w) {
    if (w.d_raw) rt->device_free(w.d_raw);
    w.d_raw = nullptr;
  };
  if (tiled) {
    dec->t_qkv.assign(L, nullptr); dec->t_o.assign(L, nullptr); dec->t_gu.assign(L, nullptr); dec->t_down.assign(L, nullptr);
    for (size_t l = 0; l < L; ++l) {
      const void* qkv_parts[3] = {dec->wq[l].d_raw, dec->wk[l].d_raw, dec->wv[l].d_raw};
      const int64_t qkv_rows[3] = {dec->wq[l].rows, dec->wk[l].rows, dec->wv[l].rows};
      const int qkv_codecs[3] = {dec->wq[l].codec, dec->wk[l].codec, dec->wv[l].codec};
      ETC_TRY(build_qweight(rt, dec->wq[l].codec, qkv_parts, qkv_rows, 3, c.d_model, 0, 1, &dec->t_qkv[l], qkv_codecs));
      const void* o_parts[1] = {dec->wo[l].d_raw};
      const int64_t o_rows[1] = {dec->wo[l].rows};
      ETC_TRY(build_qweight(rt, dec->wo[l].codec, o_parts, o_rows, 1, dec->wo[l].columns, 0, 1, &dec->t_o[l]));
      const void* gu_parts[2] = {dec->gate[l].d_raw, dec->up[l].d_raw};
      const int64_t gu_rows[2] = {dec->gate[l].rows, dec->up[l].rows};
      ETC_TRY(build_qweight(rt, dec->gate[l].codec, gu_parts, gu_rows, 2, c.d_model, 1, 1, &dec->t_gu[l]));
      const void* d_parts[1] = {dec->down[l].d_raw};
      const int64_t d_rows[1] = {dec->down[l].rows};
      ETC_TRY(build_qweight(rt, dec->down[l].codec, d_parts, d_rows, 1, dec->down[l].columns, 0, 1, &dec->t_down[l]));
      release_raw(dec->wq[l]); release_raw(dec->wk[l]); release_raw(dec->wv[l]); release_raw(dec->wo[l]);
      release_raw(dec->gate[l]); release_raw(dec->up[l]); release_raw(dec->down[l]);
    }
    const void* h_parts[1] = {dec->head.d_raw};
    const int64_t h_rows[1] = {dec->head.rows};
    ETC_TRY(build_qweight(rt, dec->head.codec, h_parts, h_rows, 1, c.d_model, 0, 1, &dec->t_head));
    release_raw(dec->head);
  }
  dec->weight_bytes = rt->memory_bytes.load();
  ETC_TRY(make_inv_freq(rt, c.rope_theta, c.head_dim, &dec->d_inv_freq));

  const size_t R = (size_t)c.batch * (size_t)dec->max_advance;
  const size_t qw = (size_t)c.q_heads * c.head_dim, kvw = (size_t)c.kv_heads * c.head_dim;
  ETC_TRY(dalloc(dec, &dec->hidden, R * c.d_model));
  ETC_TRY(dalloc(dec, &dec->normed, R * c.d_model));
  ETC_TRY(dalloc(dec, &dec->qkv, R * (qw + 2 * kvw)));
  ETC_TRY(dalloc(dec, &dec->qh, R * qw));
  ETC_TRY(dalloc(dec, &dec->kh, R * kvw));
  ETC_TRY(dalloc(dec, &dec->vh, R * kvw));
  ETC_TRY(dalloc(dec, &dec->qr, R * qw));
  ETC_TRY(dalloc(dec, &dec->kr, R * kvw));
  ETC_TRY(dalloc(dec, &dec->att, R * qw));
  ETC_TRY(dalloc(dec, &dec->attl, R * qw));
  ETC_TRY(dalloc(dec, &dec->proj, R * std::max<size_t>(c.d_model, 1)));
  ETC_TRY(dalloc(dec, &dec->g, R * c.ffn));
  ETC_TRY(dalloc(dec, &dec->u, R * c.ffn));
  ETC_TRY(dalloc(dec, &dec->act, R * c.ffn));
  ETC_TRY(dalloc(dec, &dec->last, (size_t)c.batch * c.d_model));
  ETC_TRY(dalloc(dec, &dec->logits, (size_t)c.batch * c.vocab));
  ETC_TRY(dalloc(dec, &dec->d_ids, R));
  ETC_TRY(dalloc(dec, &dec->d_cursors, (size_t)c.batch));
  ETC_TRY(dalloc(dec, &dec->d_tokens, (size_t)c.batch));
  ETC_TRY(dalloc(dec, &dec->d_step_counter, 1));
  ETC_TRY(dalloc(dec, &dec->d_lanes, (size_t)c.batch));
  dec->max_blocks = decoder_max_blocks(c, dec->max_advance);
  ETC_TRY(dalloc(dec, &dec->d_tables, (size_t)c.batch * dec->max_blocks));
  if (tiled) {
    size_t need = 0;
    // the plan (vector padding, split count) changes at these vector counts; cover every one up to R rows
    const int64_t probes[] = {1, 9, 17, 32, 64, 128, 256, (int64_t)R};
    for (size_t l = 0; l < L; ++l)
      for (etc_qweight* w : {dec->t_qkv[l], dec->t_o[l], dec->t_gu[l], dec->t_down[l]})
        for (int64_t v : probes)
          need = std::max(need, tiled_scratch_bytes(w->tiled, std::min<int64_t>(v, (int64_t)R), rt->sm_count));
    for (int64_t v : probes)
      need = std::max(need, tiled_scratch_bytes(dec->t_head->tiled, std::min<int64_t>(v, c.batch), rt->sm_count));
    dec->xh_nv = hand_off_stride(c.batch) ? hand_off_stride(c.batch) : 32;
    dec->xh_path = hand_off_stride(c.batch) != 0 && c.d_model % 8 == 0 && c.ffn % 8 == 0 && (c.q_heads * c.head_dim) % 8 == 0 &&
                   c.d_model <= 8192;
    if (dec->xh_path) {
      const size_t nv = (size_t)dec->xh_nv;
      ETC_TRY(dalloc(dec, &dec->xh_norm, (size_t)c.d_model * nv));
      ETC_TRY(dalloc(dec, &dec->xh_att, qw * nv));
      ETC_TRY(dalloc(dec, &dec->xh_act, (size_t)c.ffn * nv));
      ETC_CUDA(cudaMemsetAsync(dec->xh_norm, 0, (size_t)c.d_model * nv * sizeof(__half), rt->stream));
      ETC_CUDA(cudaMemsetAsync(dec->xh_att, 0, qw * nv * sizeof(__half), rt->stream));
      ETC_CUDA(cudaMemsetAsync(dec->xh_act, 0, (size_t)c.ffn * nv * sizeof(__half), rt->stream));
      ETC_CUDA(cudaStreamSynchronize(rt->stream));
    }
    dec->lin_scratch_bytes = need;
    if (need) ETC_TRY(dalloc(dec, &dec->lin_scratch, need / sizeof(float)));
    const size_t attn_need = decoder_attention_reserve(c, dec->max_advance, rt->sm_count);
    dec->attn_scratch_bytes = attn_need;
    ETC_TRY(dalloc(dec, &dec->attn_scratch, attn_need / sizeof(float) + 1));
  }
  cudaError_t e = cudaMallocHost((void**)&dec->h_ids, sizeof(uint32_t) * std::max<size_t>(R, 1));
  if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_cursors, sizeof(int64_t) * (size_t)c.batch);
  if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_lanes, sizeof(LaneInfo) * (size_t)c.batch);
  if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_tables, sizeof(int) * (size_t)c.batch * dec->max_blocks);
  if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_tokens, sizeof(uint32_t) * (size_t)c.batch);
  dec->h_logits_bytes = sizeof(float) * (size_t)c.batch * c.vocab;
  if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_logits, dec->h_logits_bytes);
  if (e != cudaSuccess) return fail(ETC_COMPILATION, std::string("compile: pinned staging allocation failed: ") + cudaGetErrorString(e));
  std::memset(dec->h_tables, 0, sizeof(int) * (size_t)c.batch * dec->max_blocks);
  dec->finalized = true;
  return ETC_OK;
}

etc_status etc_decoder_destroy(etc_decoder* dec) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  etc_runtime* rt = dec->rt;
  ETC_TRY(activate(rt));
  cudaStreamSynchronize(rt->stream);
  if (dec->step_graph) cudaGraphExecDestroy(dec->step_graph);
  if (dec->exec_graph) cudaGraphExecDestroy(dec->exec_graph);
  tp_comm_destroy(dec->tp);
  for (int r = 0; r < kMaxTpRanks; ++r)
    if (dec->tp_peer_base[r]) cudaIpcCloseMemHandle(dec->tp_peer_base[r]);
  if (dec->tp_region) rt->device_free(dec->tp_region);
  auto free_bound = [&](BoundWeight& w) { if (w.d_raw) rt->device_free(w.d_raw); w.d_raw = nullptr; };
  free_bound(dec->tok_embd); free_bound(dec->out_norm); free_bound(dec->head);
  for (auto* list : {&dec->attn_norm, &dec->ffn_norm, &dec->wq, &dec->wk, &dec->wv, &dec->wo, &dec->gate, &dec->up, &dec->down})
    for (auto& w : *list) free_bound(w);
  for (auto* list : {&dec->t_qkv, &dec->t_o, &dec->t_gu, &dec->t_down})
    for (etc_qweight* w : *list) destroy_qweight(w);
  destroy_qweight(dec->t_head);
  for (void* p : {(void*)dec->d_inv_freq, (void*)dec->hidden, (void*)dec->normed, (void*)dec->qkv, (void*)dec->qh, (void*)dec->kh,
                  (void*)dec->vh, (void*)dec->qr, (void*)dec->kr, (void*)dec->att, (void*)dec->attl, (void*)dec->proj, (void*)dec->g,
                  (void*)dec->u, (void*)dec->act, (void*)dec->last, (void*)dec->logits, (void*)dec->lin_scratch, (void*)dec->xh_norm,
                  (void*)dec->xh_att, (void*)dec->xh_act,
                  (void*)dec->attn_scratch, (void*)dec->exact_scratch, (void*)dec->d_ids, (void*)dec->d_cursors, (void*)dec->d_tokens,
                  (void*)dec->d_history, (void*)dec->d_step_counter, (void*)dec->d_lanes, (void*)dec->d_tables})
    if (p) rt->device_free(p);
  for (void* p : {(void*)dec->h_ids, (void*)dec->h_cursors, (void*)dec->h_lanes, (void*)dec->h_tables, (void*)dec->h_tokens, (void*)dec->h_logits})
    if (p) cudaFreeHost(p);
  dec->magic = 0;
  delete dec;
  return ETC_OK;
}

etc_status etc_decoder_execute(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active, const uint32_t* h_tokens,
                               int advance, float* h_logits, const volatile int* cancelled) {
  return execute_impl(dec, pool, seqs, active, h_tokens, advance, h_logits, nullptr, cancelled);
}

etc_status etc_decoder_execute_sampled(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active,
                                       const uint32_t* h_tokens, int advance, uint32_t* h_out_tokens,
                                       const volatile int* cancelled) {
  if (!h_out_tokens) return fail(ETC_INVALID_ARGUMENT, "executeSampled: output token buffer is null");
  return execute_impl(dec, pool, seqs, active, h_tokens, advance, nullptr, h_out_tokens, cancelled);
}

etc_status etc_decoder_generate_greedy(etc_decoder* dec, etc_pool* pool, etc_seq* const* seqs, int active,
                                       const uint32_t* h_first_tokens, int steps, uint32_t* h_out_tokens, float* out_device_ms) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  etc_runtime* rt = dec->rt;
  ETC_TRY(activate(rt));
  if (steps <= 0) return fail(ETC_INVALID_ARGUMENT, "generate: steps must be positive");
  const etc_decoder_config& c = dec->cfg;
  Transaction tx;
  StepContext ctx{};
  // pages for the whole run are reserved up front so no host work is needed between steps
  ETC_TRY(begin(dec, pool, seqs, active, h_first_tokens, 1, steps, tx, ctx));
  auto abort_with = [&](etc_status st) {
    const std::string message = last_error();
    cudaStreamSynchronize(rt->stream);
    tx.rollback();
    return fail(st, message);
  };
  if (uses_exact_attention(dec, pool, 1)) {
    etc_status st = ensure_exact_scratch(dec, ctx);
    if (st != ETC_OK) return abort_with(st);
  }
  if ((size_t)steps * c.batch > dec->history_capacity) {
    if (dec->d_history) rt->device_free(dec->d_history);
    dec->d_history = nullptr;
    void* p = nullptr;
    etc_status st = rt->device_alloc(sizeof(uint32_t) * (size_t)steps * c.batch, &p);
    if (st != ETC_OK) return abort_with(st);
    dec->d_history = (uint32_t*)p;
    dec->history_capacity = (size_t)steps * c.batch;
  }
  etc_status st = upload_step_inputs(dec, 1);
  if (st != ETC_OK) return abort_with(st);
  cudaError_t e = cudaMemsetAsync(dec->d_step_counter, 0, sizeof(int), rt->stream);
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  if (e == cudaSuccess) e = cudaEventCreate(&ev0);
  if (e == cudaSuccess) e = cudaEventCreate(&ev1);
  if (e != cudaSuccess) {
    fail(ETC_EXECUTION, std::string("generate: ") + cudaGetErrorString(e));
    return abort_with(ETC_EXECUTION);
  }
  // Step 0 runs eagerly (it also configures kernel attributes); the same launch sequence is then
  // captured once into a CUDA graph and replayed for the remaining steps. The final context of the
  // run bounds the split plan, so the captured plan is valid for every replayed step.
  const int final_pages = ctx.max_pages;
  ctx.max_ctx = std::max(ctx.max_ctx, 1);
  cudaEventRecord(ev0, rt->stream);
  auto one_step = [&]() -> etc_status {
    StepContext sc = ctx;
    sc.launches = 0;
    sc.max_pages = final_pages;
    ETC_TRY(enqueue_step(sc));
    ETC_CUDA(launch_record_step(dec->d_tokens, dec->d_ids, dec->d_history, dec->d_step_counter, dec->d_lanes, dec->d_cursors,
                                c.batch, c.window, rt->stream));
    dec->launches_last_step = sc.launches + 1;
    return ETC_OK;
  };
  st = one_step();
  if (st != ETC_OK) return abort_with(st);
  if (steps > 1) {
    if (dec->step_graph && (dec->graph_active != active || dec->graph_pages != final_pages || dec->graph_ctx != ctx.max_ctx ||
                            dec->graph_pool_uid != pool->uid)) {
      cudaGraphExecDestroy(dec->step_graph);
      dec->step_graph = nullptr;
    }
    if (!dec->step_graph) {
      cudaGraph_t graph = nullptr;
      e = cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeThreadLocal);
      if (e == cudaSuccess) {
        st = one_step();
        cudaError_t e2 = cudaStreamEndCapture(rt->stream, &graph);
        if (st == ETC_OK && e2 != cudaSuccess) e = e2;
      }
      if (st == ETC_OK && e == cudaSuccess) e = cudaGraphInstantiate(&dec->step_graph, graph, 0);
      if (graph) cudaGraphDestroy(graph);
      if (st != ETC_OK) return abort_with(st);
      if (e != cudaSuccess) {
        fail(ETC_EXECUTION, std::string("generate: graph capture failed: ") + cudaGetErrorString(e));
        return abort_with(ETC_EXECUTION);
      }
      dec->graph_active = active;
      dec->graph_pages = final_pages;
      dec->graph_ctx = ctx.max_ctx;
      dec->graph_pool_uid = pool->uid;
    }
    for (int sidx = 1; sidx < steps; ++sidx) {
      e = cudaGraphLaunch(dec->step_graph, rt->stream);
      if (e != cudaSuccess) {
        fail(ETC_EXECUTION, std::string("generate: graph launch failed: ") + cudaGetErrorString(e));
        return abort_with(ETC_EXECUTION);
      }
    }
  }
  rt->launches += (uint64_t)dec->launches_last_step * (uint64_t)steps;
  cudaEventRecord(ev1, rt->stream);
  std::vector<uint32_t> history((size_t)steps * c.batch);
  e = cudaMemcpyAsync(history.data(), dec->d_history, sizeof(uint32_t) * history.size(), cudaMemcpyDeviceToHost, rt->stream);
  if (e != cudaSuccess) {
    fail(ETC_TRANSFER, std::string("readback failed: ") + cudaGetErrorString(e));
    return abort_with(ETC_TRANSFER);
  }
  st = rt->check_status();
  float ms = 0.0f;
  cudaEventElapsedTime(&ms, ev0, ev1);
  cudaEventDestroy(ev0);
  cudaEventDestroy(ev1);
  if (st != ETC_OK) return abort_with(st);
  if (out_device_ms) *out_device_ms = ms;
  // commit every step: the token fed at step s is the first token (s = 0) or step s-1's output
  for (int i = 0; i < active; ++i) {
    etc_seq* s = seqs[i];
    std::vector<uint32_t> fed((size_t)steps);
    fed[0] = h_first_tokens[i];
    for (int sidx = 1; sidx < steps; ++sidx) fed[(size_t)sidx] = history[(size_t)(sidx - 1) * c.batch + i];
    for (int sidx = 0; sidx < steps; ++sidx) {
      if (c.window >= 0) {
        const size_t needed = s->cursor + 1;
        s->evict(needed > (size_t)c.window ? needed - (size_t)c.window : 0);
      }
      s->note_tokens(&fed[(size_t)sidx], 1);
      s->cursor += 1;
    }
    s->advance = 0;
    if (h_out_tokens)
      for (int sidx = 0; sidx < steps; ++sidx) h_out_tokens[(size_t)sidx * active + i] = history[(size_t)sidx * c.batch + i];
  }
  return ETC_OK;
}

etc_status etc_decoder_diagnostics(etc_decoder* dec, int* launches_per_step, uint64_t* weight_bytes, uint64_t* workspace_bytes) {
  if (!valid_decoder(dec)) return fail(ETC_INVALID_HANDLE, "decoder handle is invalid or destroyed");
  if (launches_per_step) *launches_per_step = dec->launches_last_step;
  if (weight_bytes) *weight_bytes = dec->weight_bytes;
  if (workspace_bytes) *workspace_bytes = dec->workspace_bytes;
  return ETC_OK;
}

}  // extern "C"
