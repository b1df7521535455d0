// Paged KV pool, sequences and the stand-alone KvAttention entry point of the C ABI.
// The allocator, prefix cache and transaction rules restate the reference's integer logic
// (crates/runtime-cpu/src/napi/mod.rs:2378-2651, 3568-3622, 3632-3947) so that page tables,
// hashes and error texts match it exactly.
#include "pool.h"

#include <algorithm>
#include <cstring>

namespace etc {

uint64_t chain_hash(uint64_t previous, const uint32_t* tokens, size_t count) {  // napi/mod.rs:2381-2390
  uint64_t hash = previous;
  for (size_t i = 0; i < count; ++i)
    for (int byte = 0; byte < 4; ++byte) {
      hash ^= (uint64_t)((tokens[i] >> (8 * byte)) & 0xff);
      hash *= kHashPrime;
    }
  return hash;
}

void BlockStore::init(size_t blocks) {
  free_list.resize(blocks);
  for (size_t i = 0; i < blocks; ++i) free_list[i] = (uint32_t)(blocks - 1 - i);  // popped from the back: 0,1,2,...
  refcounts.assign(blocks, 0);
  has_hash.assign(blocks, 0);
  hashes.assign(blocks, 0);
}
bool BlockStore::is_cached(uint32_t block) const {
  if (refcounts[block] != 0 || !has_hash[block]) return false;
  auto it = by_hash.find(hashes[block]);
  return it != by_hash.end() && std::find(it->second.begin(), it->second.end(), block) != it->second.end();
}
void BlockStore::uncache(uint32_t block, uint64_t hash) {
  auto it = by_hash.find(hash);
  if (it == by_hash.end()) return;
  auto& list = it->second;
  auto pos = std::find(list.begin(), list.end(), block);
  if (pos != list.end()) {
    *pos = list.back();
    list.pop_back();
  }
  if (list.empty()) by_hash.erase(it);
}
size_t BlockStore::cached() const {
  size_t n = 0;
  for (const auto& kv : by_hash)
    for (uint32_t b : kv.second) n += refcounts[b] == 0;
  return n;
}
long long BlockStore::alloc_block() {  // :2516-2534 — free list first, then the LRU of cached blocks
  if (!free_list.empty()) {
    const uint32_t b = free_list.back();
    free_list.pop_back();
    refcounts[b] = 1;
    has_hash[b] = 0;
    return b;
  }
  while (!lru.empty()) {
    const uint32_t candidate = lru.front();
    lru.pop_front();
    if (!is_cached(candidate)) continue;
    uncache(candidate, hashes[candidate]);
    has_hash[candidate] = 0;
    refcounts[candidate] = 1;
    return candidate;
  }
  return -1;
}
long long BlockStore::take_block(uint64_t hash) {  // :2536-2541
  auto it = by_hash.find(hash);
  if (it == by_hash.end() || it->second.empty()) return -1;
  const uint32_t b = it->second.front();
  refcounts[b] += 1;
  return b;
}
void BlockStore::unref_block(uint32_t block) {  // :2543-2554
  uint32_t& count = refcounts[block];
  if (count > 0) --count;
  if (count == 0) {
    if (has_hash[block]) lru.push_back(block);
    else free_list.push_back(block);
  }
}
void BlockStore::set_hash(uint32_t block, uint64_t hash) {  // :2556-2561
  has_hash[block] = 1;
  hashes[block] = hash;
  by_hash[hash].push_back(block);
}

etc_status kv_prepare(etc_pool* pool, etc_seq* seq, int layer, int64_t pool_window, int heads, int width, int tokens,
                      size_t* cursor, size_t* needed, size_t* start) {
  if (layer >= pool->layers)
    return fail(ETC_EXECUTION, "kv attention: layer " + std::to_string(layer) + " out of range for " +
                                   std::to_string(pool->layers) + " pool layers");
  if (heads != pool->kv_heads || width != pool->head_dim)
    return fail(ETC_EXECUTION, "kv attention: layer " + std::to_string(layer) + " shape [" + std::to_string(heads) + ", " +
                                   std::to_string(width) + "] does not match pool geometry [" +
                                   std::to_string(pool->kv_heads) + ", " + std::to_string(pool->head_dim) + "]");
  *cursor = seq->cursor;
  const size_t advance = seq->advance;
  if (advance == 0 || advance > (size_t)tokens)
    return fail(ETC_EXECUTION, "kv attention: advance " + std::to_string(advance) + " out of range for chunk length " +
                                   std::to_string(tokens));
  *needed = *cursor + advance;
  *start = pool_window >= 0 ? (*needed > (size_t)pool_window ? *needed - (size_t)pool_window : 0) : 0;
  if (*needed - *start > (size_t)pool->max_tokens)
    return fail(ETC_EXECUTION, "kv attention: live context " + std::to_string(*needed - *start) +
                                   " exceeds pool capacity " + std::to_string(pool->max_tokens));
  std::lock_guard<std::mutex> guard(pool->mutex);
  while (seq->blocks.size() * (size_t)pool->block_size < *needed) {
    const long long b = pool->store.alloc_block();
    if (b < 0)
      return fail(ETC_EXECUTION, "kv attention: pool exhausted (" + std::to_string(pool->max_tokens) +
                                     " tokens across live sequences)");
    seq->blocks.push_back((uint32_t)b);
  }
  return ETC_OK;
}

}  // namespace etc

using namespace etc;

PoolView etc_pool::view(int layer) const {
  PoolView v;
  const size_t esize = (size_t)kv_dtype_size(dtype);
  v.k = (char*)d_k + (size_t)layer * layer_elems * esize;
  v.v = (char*)d_v + (size_t)layer * layer_elems * esize;
  v.k_scale = d_k_scale ? d_k_scale + (size_t)layer * layer_scales : nullptr;
  v.v_scale = d_v_scale ? d_v_scale + (size_t)layer * layer_scales : nullptr;
  v.dtype = dtype;
  v.kv_heads = kv_heads;
  v.head_dim = head_dim;
  v.block_size = block_size;
  return v;
}

void etc_seq::note_tokens(const uint32_t* tokens, size_t count) {  // napi/mod.rs:2637-2650
  std::lock_guard<std::mutex> guard(pool->mutex);
  for (size_t i = 0; i < count; ++i) {
    pending.push_back(tokens[i]);
    if ((int)pending.size() == pool->block_size) {
      const uint64_t hash = chain_hash(last_hash, pending.data(), pending.size());
      last_hash = hash;
      pending.clear();
      const size_t block_index = (cursor + i) / (size_t)pool->block_size;
      if (block_index < blocks.size()) pool->store.set_hash(blocks[block_index], hash);
    }
  }
}
void etc_seq::evict(size_t start) {  // :3617-3622
  std::lock_guard<std::mutex> guard(pool->mutex);
  while (head < blocks.size() && (head + 1) * (size_t)pool->block_size <= start) {
    pool->store.unref_block(blocks[head]);
    head += 1;
  }
}
void etc_seq::rollback_to(size_t frontier) {  // :2888-2893
  std::lock_guard<std::mutex> guard(pool->mutex);
  for (size_t i = frontier; i < blocks.size(); ++i) pool->store.unref_block(blocks[i]);
  if (blocks.size() > frontier) blocks.resize(frontier);
  advance = 0;
}
void etc_seq::return_blocks() {  // :3825-3842
  if (released) return;
  released = true;
  std::lock_guard<std::mutex> run(run_lock);
  std::lock_guard<std::mutex> guard(pool->mutex);
  for (size_t i = head; i < blocks.size(); ++i) pool->store.unref_block(blocks[i]);
  blocks.resize(std::min(head, blocks.size()));
  cursor = 0;
  advance = 0;
  last_hash = kHashSeed;
  pending.clear();
}

static bool valid_pool(const etc_pool* p) { return p && p->magic == kPoolMagic; }
static bool valid_seq(const etc_seq* s) { return s && s->magic == kSeqMagic; }

extern "C" {

etc_status etc_pool_create(etc_runtime* rt, int layers, int kv_heads, int head_dim, int max_tokens, int block_size,
                           etc_kv_dtype dtype, etc_pool** out) {
  ETC_TRY(activate(rt));
  if (!out) return fail(ETC_INVALID_ARGUMENT, "out is null");
  *out = nullptr;
  // NativeKvPool::new geometry rules (napi/mod.rs:3651-3708)
  if (dtype < ETC_KV_F32 || dtype > ETC_KV_U8)
    return fail(ETC_INVALID_ARGUMENT, "kv pool: dtype must be f32, f16, bf16 or u8 (int8-quantized)");
  if (layers < 0 || kv_heads < 0 || head_dim < 0) return fail(ETC_INVALID_ARGUMENT, "kv pool: negative geometry");
  if (layers == 0 && (kv_heads != 0 || head_dim != 0))
    return fail(ETC_INVALID_ARGUMENT, "kv pool: heads and head dim must be zero when layers is zero");
  if (layers > 0 && (kv_heads == 0 || head_dim == 0))
    return fail(ETC_INVALID_ARGUMENT, "kv pool: layers, kv heads and head dim must be positive");
  if (block_size <= 0 || max_tokens <= 0 || max_tokens % block_size != 0)
    return fail(ETC_INVALID_ARGUMENT, "kv pool: capacity " + std::to_string(max_tokens) +
                                          " must be a positive multiple of block size " + std::to_string(block_size));
  etc_pool* p = new etc_pool();
  static std::atomic<uint64_t> next_uid{1};
  p->uid = next_uid.fetch_add(1);
  p->rt = rt;
  p->layers = layers; p->kv_heads = kv_heads; p->head_dim = head_dim;
  p->max_tokens = max_tokens; p->block_size = block_size; p->dtype = dtype;
  p->layer_elems = (size_t)max_tokens * kv_heads * head_dim;
  p->layer_scales = (size_t)max_tokens * kv_heads;
  const size_t bytes = p->layer_elems * layers * (size_t)kv_dtype_size(dtype);
  etc_status st = rt->device_alloc(bytes, &p->d_k);
  if (st == ETC_OK) st = rt->device_alloc(bytes, &p->d_v);
  if (st == ETC_OK && dtype == ETC_KV_U8) {
    st = rt->device_alloc(p->layer_scales * layers * sizeof(float), (void**)&p->d_k_scale);
    if (st == ETC_OK) st = rt->device_alloc(p->layer_scales * layers * sizeof(float), (void**)&p->d_v_scale);
  }
  if (st == ETC_OK && bytes > 0) {
    // slabs start zeroed like the reference's (pool.rs:95-112)
    cudaError_t e = cudaMemsetAsync(p->d_k, 0, bytes, rt->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->d_v, 0, bytes, rt->stream);
    if (e == cudaSuccess && p->d_k_scale) e = cudaMemsetAsync(p->d_k_scale, 0, p->layer_scales * layers * sizeof(float), rt->stream);
    if (e == cudaSuccess && p->d_v_scale) e = cudaMemsetAsync(p->d_v_scale, 0, p->layer_scales * layers * sizeof(float), rt->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
    if (e != cudaSuccess) st = fail(ETC_EXECUTION, std::string("kv pool: clearing slabs failed: ") + cudaGetErrorString(e));
  }
  if (st != ETC_OK) {
    const std::string message = last_error();
    rt->device_free(p->d_k); rt->device_free(p->d_v); rt->device_free(p->d_k_scale); rt->device_free(p->d_v_scale);
    delete p;
    return fail(st, message);
  }
  p->store.init((size_t)(max_tokens / block_size));
  *out = p;
  return ETC_OK;
}

etc_status etc_pool_destroy(etc_pool* pool) {
  if (!valid_pool(pool)) return fail(ETC_INVALID_HANDLE, "kv pool handle is invalid or destroyed");
  ETC_TRY(activate(pool->rt));
  cudaStreamSynchronize(pool->rt->stream);
  pool->rt->device_free(pool->d_k);
  pool->rt->device_free(pool->d_v);
  pool->rt->device_free(pool->d_k_scale);
  pool->rt->device_free(pool->d_v_scale);
  pool->magic = 0;
  delete pool;
  return ETC_OK;
}

etc_status etc_pool_stats(etc_pool* pool, uint32_t* capacity, uint32_t* free_blocks, uint32_t* cached_blocks) {
  if (!valid_pool(pool)) return fail(ETC_INVALID_HANDLE, "kv pool handle is invalid or destroyed");
  std::lock_guard<std::mutex> guard(pool->mutex);
  const size_t cached = pool->store.cached();
  if (capacity) *capacity = (uint32_t)pool->max_tokens;
  if (free_blocks) *free_blocks = (uint32_t)(pool->store.free_list.size() + cached);  // available(), :2611-2616
  if (cached_blocks) *cached_blocks = (uint32_t)cached;
  return ETC_OK;
}

etc_status etc_pool_state_bytes(int64_t layers, int64_t max_tokens, int64_t kv_heads, int64_t head_dim,
                                etc_kv_dtype dtype, int64_t* out_bytes) {
  const int size = kv_dtype_size(dtype);
  if (size == 0) return fail(ETC_COMPILATION, "compile: unsupported KV state dtype");
  int64_t bytes = layers * max_tokens * kv_heads * head_dim * 2 * size;
  if (dtype == ETC_KV_U8) bytes += layers * max_tokens * kv_heads * 2 * 4;
  *out_bytes = bytes;
  return ETC_OK;
}

etc_status etc_pool_read_rows(etc_pool* pool, int layer, int which, const uint32_t* h_rows, int64_t n, float* h_out) {
  if (!valid_pool(pool)) return fail(ETC_INVALID_HANDLE, "kv pool handle is invalid or destroyed");
  etc_runtime* rt = pool->rt;
  ETC_TRY(activate(rt));
  if (layer < 0 || layer >= pool->layers) return fail(ETC_INVALID_ARGUMENT, "kv pool: layer out of range");
  for (int64_t i = 0; i < n; ++i)
    if (h_rows[i] >= (uint32_t)pool->max_tokens) return fail(ETC_INVALID_ARGUMENT, "kv pool: row out of range");
  if (n == 0) return ETC_OK;
  const size_t width = (size_t)pool->kv_heads * pool->head_dim;
  void* ws = nullptr;
  const size_t rows_bytes = ((size_t)n * sizeof(uint32_t) + 255) & ~(size_t)255;
  ETC_TRY(rt->workspace(rows_bytes + (size_t)n * width * sizeof(float), &ws));
  uint32_t* d_rows = (uint32_t*)ws;
  float* d_out = (float*)((char*)ws + rows_bytes);
  ETC_CUDA(cudaMemcpyAsync(d_rows, h_rows, (size_t)n * sizeof(uint32_t), cudaMemcpyHostToDevice, rt->stream));
  ETC_CUDA(launch_pool_read_rows(pool->view(layer), d_rows, n, d_out, which, rt->stream));
  rt->launches++;
  ETC_CUDA(cudaMemcpyAsync(h_out, d_out, (size_t)n * width * sizeof(float), cudaMemcpyDeviceToHost, rt->stream));
  ETC_CUDA(cudaStreamSynchronize(rt->stream));
  return ETC_OK;
}

etc_status etc_seq_create(etc_pool* pool, etc_seq** out) {
  if (!valid_pool(pool)) return fail(ETC_INVALID_HANDLE, "kv pool handle is invalid or destroyed");
  etc_seq* s = new etc_seq();
  s->pool = pool;
  s->blocks.reserve((size_t)(pool->max_tokens / pool->block_size));
  *out = s;
  return ETC_OK;
}

etc_status etc_seq_release(etc_seq* seq) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  seq->return_blocks();
  return ETC_OK;
}

etc_status etc_seq_destroy(etc_seq* seq) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  seq->return_blocks();
  seq->magic = 0;
  delete seq;
  return ETC_OK;
}

etc_status etc_seq_cursor(etc_seq* seq, uint32_t* out_cursor) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  *out_cursor = (uint32_t)seq->cursor;
  return ETC_OK;
}

etc_status etc_seq_prefill_match(etc_seq* seq, const uint32_t* h_tokens, int64_t count, uint32_t* out_matched) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  std::lock_guard<std::mutex> run(seq->run_lock);
  if (seq->released) return fail(ETC_EXECUTION, "kv sequence is released");
  if (seq->cursor > 0 || !seq->blocks.empty()) return fail(ETC_EXECUTION, "prefill match: sequence already holds tokens");
  etc_pool* pool = seq->pool;
  const int64_t matchable = (count > 0 ? count - 1 : 0) / pool->block_size;  // :3903 — the last token always runs
  uint64_t hash = kHashSeed;
  {
    std::lock_guard<std::mutex> guard(pool->mutex);
    for (int64_t i = 0; i < matchable; ++i) {
      const uint64_t next = chain_hash(hash, h_tokens + i * pool->block_size, (size_t)pool->block_size);
      const long long b = pool->store.take_block(next);
      if (b < 0) break;
      seq->blocks.push_back((uint32_t)b);
      hash = next;
    }
  }
  seq->last_hash = hash;
  seq->cursor = seq->blocks.size() * (size_t)pool->block_size;
  if (out_matched) *out_matched = (uint32_t)seq->cursor;
  return ETC_OK;
}

etc_status etc_seq_blocks(etc_seq* seq, uint32_t* h_out, int64_t capacity, int64_t* out_count, int64_t* out_head) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  if (out_count) *out_count = (int64_t)seq->blocks.size();
  if (out_head) *out_head = (int64_t)seq->head;
  if (h_out)
    for (int64_t i = 0; i < capacity && i < (int64_t)seq->blocks.size(); ++i) h_out[i] = seq->blocks[(size_t)i];
  return ETC_OK;
}

etc_status etc_seq_frontier(etc_seq* seq, int64_t* out_frontier) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  *out_frontier = (int64_t)seq->blocks.size();
  return ETC_OK;
}

etc_status etc_seq_commit(etc_seq* seq, const uint32_t* h_tokens, int advance, int64_t eviction_start) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  if (seq->released) return fail(ETC_EXECUTION, "kv sequence is released");
  if (advance <= 0) return fail(ETC_INVALID_ARGUMENT, "kv run: expected one non-empty token list per sequence");
  if (eviction_start > 0) seq->evict((size_t)eviction_start);
  seq->note_tokens(h_tokens, (size_t)advance);
  seq->cursor += (size_t)advance;
  seq->advance = 0;
  return ETC_OK;
}

etc_status etc_seq_rollback(etc_seq* seq, int64_t frontier) {
  if (!valid_seq(seq)) return fail(ETC_INVALID_HANDLE, "kv sequence handle is invalid or destroyed");
  seq->rollback_to((size_t)std::max<int64_t>(frontier, 0));
  return ETC_OK;
}

}  // extern "C"

namespace {

// Shared host part of the stand-alone KvAttention entry points: kv_prepare per active lane, lane
// descriptors and block tables staged into the runtime workspace (followed by `extra` bytes).
struct StagedLanes {
  LaneInfo* d_lanes = nullptr;
  int* d_tables = nullptr;
  void* d_extra = nullptr;
  int max_ctx = 1;
  int max_pages = 1;
};

etc_status stage_lanes(etc_runtime* rt, etc_pool* pool, int layer, etc_seq* const* seqs, int batch, int active, int advance,
                       int tokens, int64_t pool_window, size_t extra_bytes_per_ctx, size_t extra_fixed, StagedLanes* out) {
  if (!valid_pool(pool) || pool->rt != rt) return fail(ETC_INVALID_HANDLE, "kv pool belongs to a different runtime");
  if (batch <= 0 || active < 0 || active > batch) return fail(ETC_INVALID_ARGUMENT, "kv attention: invalid batch");
  for (int i = 0; i < active; ++i) {
    if (!valid_seq(seqs[i]) || seqs[i]->pool != pool) return fail(ETC_INVALID_HANDLE, "kv sequence does not belong to this pool");
    if (seqs[i]->released) return fail(ETC_EXECUTION, "kv sequence " + std::to_string(i) + " is released");
  }
  std::vector<LaneInfo> lanes((size_t)batch);
  std::vector<int> tables;
  for (int i = 0; i < batch; ++i) {
    LaneInfo info{0, 0, 0, 0};
    if (i < active) {
      etc_seq* s = seqs[i];
      s->advance = (size_t)advance;
      size_t cursor, needed, start;
      ETC_TRY(kv_prepare(pool, s, layer, pool_window, pool->kv_heads, pool->head_dim, tokens, &cursor, &needed, &start));
      info.cursor = (int)cursor;
      info.advance = advance;
      info.start = (int)start;
      info.table_offset = (int)tables.size();
      for (uint32_t b : s->blocks) tables.push_back((int)b);
      out->max_ctx = std::max(out->max_ctx, (int)(needed - start));
      out->max_pages = std::max(out->max_pages, (int)((needed + pool->block_size - 1) / pool->block_size) - (int)(start / pool->block_size));
    }
    lanes[(size_t)i] = info;
  }
  if (tables.empty()) tables.push_back(0);
  const size_t lanes_bytes = (lanes.size() * sizeof(LaneInfo) + 255) & ~(size_t)255;
  const size_t tables_bytes = (tables.size() * sizeof(int) + 255) & ~(size_t)255;
  const size_t extra = extra_bytes_per_ctx * (size_t)out->max_ctx + extra_fixed;
  void* ws = nullptr;
  ETC_TRY(rt->workspace(lanes_bytes + tables_bytes + extra, &ws));
  out->d_lanes = (LaneInfo*)ws;
  out->d_tables = (int*)((char*)ws + lanes_bytes);
  out->d_extra = (char*)ws + lanes_bytes + tables_bytes;
  ETC_CUDA(cudaMemcpyAsync(out->d_lanes, lanes.data(), lanes.size() * sizeof(LaneInfo), cudaMemcpyHostToDevice, rt->stream));
  ETC_CUDA(cudaMemcpyAsync(out->d_tables, tables.data(), tables.size() * sizeof(int), cudaMemcpyHostToDevice, rt->stream));
  return ETC_OK;
}

}  // namespace

extern "C" {

etc_status etc_kv_append_into(etc_runtime* rt, etc_pool* pool, int layer, etc_seq* const* seqs, int batch, int active,
                              int advance, const float* d_k, const float* d_v, int tokens, int64_t pool_window) {
  ETC_TRY(activate(rt));
  StagedLanes st;
  ETC_TRY(stage_lanes(rt, pool, layer, seqs, batch, active, advance, tokens, pool_window, 0, 0, &st));
  const int D = pool->head_dim, Hkv = pool->kv_heads;
  ETC_CUDA(launch_kv_append(pool->view(layer), d_k, d_v, st.d_lanes, st.d_tables, batch, tokens, (int64_t)Hkv * tokens * D,
                            (int64_t)tokens * D, D, rt->stream));
  rt->launches++;
  ETC_CUDA(cudaStreamSynchronize(rt->stream));
  return ETC_OK;
}

etc_status etc_kv_attention_into(etc_runtime* rt, etc_pool* pool, int layer, etc_seq* const* seqs, int batch, int active,
                                 int advance, const float* d_q, const float* d_k, const float* d_v, int q_heads,
                                 int tokens, double scale, int64_t op_window, int64_t pool_window, float* d_out) {
  ETC_TRY(activate(rt));
  if (!valid_pool(pool)) return fail(ETC_INVALID_HANDLE, "kv pool handle is invalid or destroyed");
  if (pool->kv_heads == 0 || q_heads % pool->kv_heads != 0)
    return fail(ETC_EXECUTION, "kv attention: incompatible grouped-query q/k/v shapes");
  const int D = pool->head_dim, Hkv = pool->kv_heads;
  const size_t rows = (size_t)batch * q_heads * tokens;
  StagedLanes st;
  ETC_TRY(stage_lanes(rt, pool, layer, seqs, batch, active, advance, tokens, pool_window, rows * sizeof(double), 0, &st));
  const PoolView view = pool->view(layer);
  // scatter: k/v are [B,Hkv,T,D]
  ETC_CUDA(launch_kv_append(view, d_k, d_v, st.d_lanes, st.d_tables, batch, tokens, (int64_t)Hkv * tokens * D, (int64_t)tokens * D, D,
                            rt->stream));
  rt->launches++;
  ETC_CUDA(launch_attention_exact(view, d_q, st.d_lanes, st.d_tables, batch, q_heads, tokens, scale, op_window, d_out,
                                  (double*)st.d_extra, st.max_ctx, rt->stream));
  rt->launches++;
  // the staging buffers are reused by the next call: finish before returning
  ETC_CUDA(cudaStreamSynchronize(rt->stream));
  return ETC_OK;
}

etc_status etc_kv_attention_decode_into(etc_runtime* rt, etc_pool* pool, int layer, etc_seq* const* seqs, int batch, int active,
                                        const float* d_q, const float* d_k, const float* d_v, int q_heads, double scale,
                                        int64_t op_window, int64_t pool_window, float* d_out) {
  ETC_TRY(activate(rt));
  if (!valid_pool(pool)) return fail(ETC_INVALID_HANDLE, "kv pool handle is invalid or destroyed");
  if (pool->kv_heads == 0 || q_heads % pool->kv_heads != 0)
    return fail(ETC_EXECUTION, "kv attention: incompatible grouped-query q/k/v shapes");
  const PoolView view = pool->view(layer < pool->layers ? layer : 0);
  if (!attention_mma_supported(view, q_heads, 1))
    return fail(ETC_UNSUPPORTED, "kv attention: the tensor-core decode kernel needs an f16/bf16 pool with 16-token pages, head "
                                 "dim 64 or 128 and at most 16 query heads per kv head");
  const int D = pool->head_dim, Hkv = pool->kv_heads;
  const size_t max_scratch = plan_attention_max_scratch(batch, q_heads, Hkv, D, pool->max_tokens / pool->block_size, rt->sm_count);
  StagedLanes st;
  ETC_TRY(stage_lanes(rt, pool, layer, seqs, batch, active, 1, 1, pool_window, 0, max_scratch + 256, &st));
  float* scratch = (float*)(((uintptr_t)st.d_extra + 255) & ~(uintptr_t)255);
  if (d_k && d_v) {
    ETC_CUDA(launch_kv_append(view, d_k, d_v, st.d_lanes, st.d_tables, batch, 1, (int64_t)Hkv * D, (int64_t)D, D, rt->stream));
    rt->launches++;
  }
  const AttnPlan plan = plan_attention(batch, q_heads, Hkv, D, st.max_pages, rt->sm_count);
  int launches = 0;
  ETC_CUDA(launch_attention_mma(view, d_q, st.d_lanes, st.d_tables, batch, q_heads, scale, op_window, d_out, plan, scratch,
                                rt->stream, &launches));
  rt->launches += (uint64_t)launches;
  ETC_CUDA(cudaStreamSynchronize(rt->stream));
  return ETC_OK;
}

etc_status etc_paged_attention_into(etc_runtime* rt, etc_pool* pool, int layer, const etc_lane* d_lanes, const int* d_tables,
                                    int batch, int max_pages, const float* d_q, int q_heads, double scale, int64_t op_window,
                                    float* d_out, void* d_scratch, size_t scratch_bytes) {
  ETC_TRY(activate(rt));
  if (!valid_pool(pool) || pool->rt != rt) return fail(ETC_INVALID_HANDLE, "kv pool belongs to a different runtime");
  if (layer < 0 || layer >= pool->layers) return fail(ETC_INVALID_ARGUMENT, "kv attention: layer index out of range");
  if (batch <= 0 || max_pages <= 0 || !d_lanes || !d_tables || !d_q || !d_out)
    return fail(ETC_INVALID_ARGUMENT, "kv attention: lanes, tables, q and out must be given for a positive batch and page bound");
  if (pool->kv_heads == 0 || q_heads % pool->kv_heads != 0)
    return fail(ETC_EXECUTION, "kv attention: incompatible grouped-query q/k/v shapes");
  const PoolView view = pool->view(layer);
  if (!attention_mma_supported(view, q_heads, 1))
    return fail(ETC_UNSUPPORTED, "kv attention: the tensor-core decode kernel needs an f16/bf16 pool with 16-token pages, head "
                                 "dim 64 or 128 and at most 16 query heads per kv head");
  static_assert(sizeof(etc_lane) == sizeof(LaneInfo), "etc_lane is the kernel's lane descriptor");
  const AttnPlan plan = plan_attention(batch, q_heads, pool->kv_heads, pool->head_dim, max_pages, rt->sm_count);
  if (plan.scratch_bytes > scratch_bytes || (plan.scratch_bytes && !d_scratch))
    return fail(ETC_INVALID_ARGUMENT, "kv attention: scratch holds " + std::to_string(scratch_bytes) + " bytes, " +
                                          std::to_string(plan.scratch_bytes) + " needed");
  int launches = 0;
  ETC_CUDA(launch_attention_mma(view, d_q, reinterpret_cast<const LaneInfo*>(d_lanes), d_tables, batch, q_heads, scale, op_window,
                                d_out, plan, reinterpret_cast<float*>(d_scratch), rt->stream, &launches));
  rt->launches += (uint64_t)launches;
  return ETC_OK;
}

}  // extern "C"
