// Host-side vocabulary shared by the C-ABI translation units: status/error plumbing, the
// runtime object and CUDA call checking. Mirrors the error classes of the reference's
// BackendError (crates/runtime/src/error.rs:25-68).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/et_cuda.h"

namespace etc {

// Thread-local last error text (returned by etc_last_error_message).
std::string& last_error();
etc_status fail(etc_status status, const std::string& message);

#define ETC_CUDA(call)                                                                              \
  do {                                                                                              \
    cudaError_t err__ = (call);                                                                     \
    if (err__ != cudaSuccess)                                                                       \
      return ::etc::fail(ETC_EXECUTION, std::string(#call) + ": " + cudaGetErrorString(err__));     \
  } while (0)

#define ETC_TRY(expr)                     \
  do {                                    \
    etc_status st__ = (expr);             \
    if (st__ != ETC_OK) return st__;      \
  } while (0)

// Device-side status word. Kernels record the first problem they see with one atomicCAS on
// `code`; the host reads it at synchronising calls and turns it into ETC_EXECUTION.
struct DeviceStatus {
  unsigned long long code;     // 0 none, 1 embedding index out of range, 2 non-finite logit
  long long value;             // offending index / token position
  long long bound;             // rows / vocabulary
  long long reserved;
};
enum : unsigned long long { kStatusNone = 0, kStatusIndexOutOfRange = 1, kStatusNonFiniteLogit = 2 };

constexpr uint32_t kRuntimeMagic = 0x45544352;  // "ETCR"
constexpr uint32_t kPoolMagic = 0x45544350;
constexpr uint32_t kSeqMagic = 0x45544353;
constexpr uint32_t kWeightMagic = 0x45544357;
constexpr uint32_t kDecoderMagic = 0x45544344;

}  // namespace etc

// The runtime owns a device ordinal, one stream, the status word and a growable workspace.
struct etc_runtime {
  uint32_t magic = etc::kRuntimeMagic;
  uint64_t id = 0;  // RuntimeId: handles remember it and foreign handles are rejected
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  etc::DeviceStatus* d_status = nullptr;
  etc::DeviceStatus* h_status = nullptr;  // pinned
  uint32_t* d_sampled = nullptr;          // one token: etc_sample_row's device output and its pinned copy
  uint32_t* h_sampled = nullptr;
  void* d_workspace = nullptr;
  size_t workspace_bytes = 0;
  std::atomic<uint64_t> launches{0};
  std::atomic<uint64_t> memory_bytes{0};
  std::mutex mutex;
  std::unordered_map<void*, size_t> allocations;

  // Grows the shared scratch workspace (never during graph capture); returns the pointer.
  etc_status workspace(size_t bytes, void** out);
  etc_status device_alloc(size_t bytes, void** out);
  etc_status device_free(void* ptr);
  // Reads the status word (after the caller synchronised) and clears it.
  etc_status check_status();
};

namespace etc {
inline bool valid(const etc_runtime* rt) { return rt && rt->magic == kRuntimeMagic; }
etc_status activate(etc_runtime* rt);  // cudaSetDevice + handle validation
const char* codec_name(int codec);
int codec_block_values(int codec);
int codec_block_bytes(int codec);
int64_t codec_row_bytes(int codec, int64_t columns);  // -1 when invalid
int kv_dtype_size(int dtype);
}  // namespace etc
