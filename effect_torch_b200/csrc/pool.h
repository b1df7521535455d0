// Host-side paged-KV state: the page allocator with its prefix cache, sequences, and the device
// slabs of a pool. Integer logic follows the reference exactly (crates/runtime-cpu/src/napi/mod.rs:
// BlockStore/PoolInner :2444-2621, SeqState :2623-2651, kv_prepare/kv_evict :3568-3622,
// NativeKvPool/NativeKvSequence :3632-3947) so page tables are identical for identical call
// sequences.
#pragma once

#include <deque>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "kernels.h"

namespace etc {

constexpr uint64_t kHashSeed = 0xcbf29ce484222325ull;
constexpr uint64_t kHashPrime = 0x00000100000001b3ull;
uint64_t chain_hash(uint64_t previous, const uint32_t* tokens, size_t count);

struct BlockStore {
  std::vector<uint32_t> free_list;
  std::vector<uint32_t> refcounts;
  std::vector<uint8_t> has_hash;
  std::vector<uint64_t> hashes;
  std::unordered_map<uint64_t, std::vector<uint32_t>> by_hash;
  std::deque<uint32_t> lru;

  void init(size_t blocks);
  bool is_cached(uint32_t block) const;
  void uncache(uint32_t block, uint64_t hash);
  size_t cached() const;
  long long alloc_block();
  long long take_block(uint64_t hash);
  void unref_block(uint32_t block);
  void set_hash(uint32_t block, uint64_t hash);
};

}  // namespace etc

struct etc_pool {
  uint32_t magic = etc::kPoolMagic;
  uint64_t uid = 0;  // process-wide serial number: captured graphs key on it, never on the handle's address
  etc_runtime* rt = nullptr;
  int layers = 0, kv_heads = 0, head_dim = 0, max_tokens = 0, block_size = 0, dtype = 0;
  size_t layer_elems = 0;   // elements per layer slab
  size_t layer_scales = 0;  // scale entries per layer (u8 tier)
  void* d_k = nullptr;      // [layers][pages][kv_heads][block_size][head_dim]
  void* d_v = nullptr;
  float* d_k_scale = nullptr;
  float* d_v_scale = nullptr;
  std::mutex mutex;         // guards the block store
  etc::BlockStore store;
  etc::PoolView view(int layer) const;
};

struct etc_seq {
  uint32_t magic = etc::kSeqMagic;
  etc_pool* pool = nullptr;
  std::vector<uint32_t> blocks;
  size_t head = 0, cursor = 0, advance = 0;
  uint64_t last_hash = etc::kHashSeed;
  std::vector<uint32_t> pending;
  bool released = false;
  std::mutex run_lock;

  void note_tokens(const uint32_t* tokens, size_t count);
  void evict(size_t start);
  void rollback_to(size_t frontier);
  void return_blocks();
};

namespace etc {
// kv_prepare (napi/mod.rs:3568-3615): validates advance/capacity and allocates pages up to
// cursor+advance. Returns ETC_OK or ETC_EXECUTION with the reference's message.
etc_status kv_prepare(etc_pool* pool, etc_seq* seq, int layer, int64_t pool_window, int heads, int width, int tokens,
                      size_t* cursor, size_t* needed, size_t* start);
}  // namespace etc
