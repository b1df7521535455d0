// Runtime object, error plumbing and device buffers of the C ABI.
#include <cuda_fp16.h>

#include <atomic>
#include <cstring>

#include "common.h"
#include "weights.h"

namespace etc {

std::string& last_error() {
  thread_local std::string message;
  return message;
}

etc_status fail(etc_status status, const std::string& message) {
  last_error() = message;
  return status;
}

etc_status activate(etc_runtime* rt) {
  if (!valid(rt)) return fail(ETC_INVALID_HANDLE, "runtime handle is invalid or destroyed");
  cudaError_t e = cudaSetDevice(rt->device);
  if (e != cudaSuccess) return fail(ETC_UNAVAILABLE, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  return ETC_OK;
}

const char* codec_name(int codec) {
  switch (codec) {
    case ETC_CODEC_F32: return "F32";
    case ETC_CODEC_Q4_0: return "Q4_0";
    case ETC_CODEC_Q8_0: return "Q8_0";
    case ETC_CODEC_Q2_K: return "Q2_K";
    case ETC_CODEC_Q3_K: return "Q3_K";
    case ETC_CODEC_Q4_K: return "Q4_K";
    case ETC_CODEC_Q5_K: return "Q5_K";
    case ETC_CODEC_Q6_K: return "Q6_K";
    default: return "unknown";
  }
}
int codec_block_values(int codec) {
  switch (codec) {
    case ETC_CODEC_Q4_0: case ETC_CODEC_Q8_0: return 32;
    case ETC_CODEC_Q2_K: case ETC_CODEC_Q3_K: case ETC_CODEC_Q4_K: case ETC_CODEC_Q5_K: case ETC_CODEC_Q6_K: return 256;
    default: return 0;
  }
}
int codec_block_bytes(int codec) {
  switch (codec) {
    case ETC_CODEC_Q4_0: return 18;
    case ETC_CODEC_Q8_0: return 34;
    case ETC_CODEC_Q2_K: return 84;
    case ETC_CODEC_Q3_K: return 110;
    case ETC_CODEC_Q4_K: return 144;
    case ETC_CODEC_Q5_K: return 176;
    case ETC_CODEC_Q6_K: return 210;
    default: return 0;
  }
}
int64_t codec_row_bytes(int codec, int64_t columns) {
  const int values = codec_block_values(codec);
  if (values == 0 || columns < 0 || columns % values != 0) return -1;
  return columns / values * codec_block_bytes(codec);
}
int kv_dtype_size(int dtype) {
  switch (dtype) {
    case ETC_KV_F32: return 4;
    case ETC_KV_F16: case ETC_KV_BF16: return 2;
    case ETC_KV_U8: return 1;
    default: return 0;
  }
}

}  // namespace etc

using namespace etc;

etc_status etc_runtime::device_alloc(size_t bytes, void** out) {
  *out = nullptr;
  if (bytes == 0) return ETC_OK;
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ETC_EXECUTION, "device allocation of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e));
  }
  {
    std::lock_guard<std::mutex> guard(mutex);
    allocations[ptr] = bytes;
  }
  memory_bytes += bytes;
  *out = ptr;
  return ETC_OK;
}

etc_status etc_runtime::device_free(void* ptr) {
  if (!ptr) return ETC_OK;
  size_t bytes = 0;
  {
    std::lock_guard<std::mutex> guard(mutex);
    auto it = allocations.find(ptr);
    if (it == allocations.end()) return fail(ETC_INVALID_HANDLE, "buffer does not belong to this runtime or was already released");
    bytes = it->second;
    allocations.erase(it);
  }
  memory_bytes -= bytes;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(ETC_EXECUTION, std::string("cudaFree: ") + cudaGetErrorString(e));
  return ETC_OK;
}

etc_status etc_runtime::workspace(size_t bytes, void** out) {
  if (bytes > workspace_bytes) {
    // Growing replaces the buffer: wait for work that may still use the old one.
    ETC_CUDA(cudaStreamSynchronize(stream));
    if (d_workspace) ETC_TRY(device_free(d_workspace));
    d_workspace = nullptr;
    workspace_bytes = 0;
    const size_t rounded = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    ETC_TRY(device_alloc(rounded, &d_workspace));
    workspace_bytes = rounded;
  }
  *out = d_workspace;
  return ETC_OK;
}

etc_status etc_runtime::check_status() {
  ETC_CUDA(cudaMemcpyAsync(h_status, d_status, sizeof(DeviceStatus), cudaMemcpyDeviceToHost, stream));
  ETC_CUDA(cudaStreamSynchronize(stream));
  if (h_status->code == kStatusNone) return ETC_OK;
  const DeviceStatus seen = *h_status;
  ETC_CUDA(cudaMemsetAsync(d_status, 0, sizeof(DeviceStatus), stream));
  ETC_CUDA(cudaStreamSynchronize(stream));
  if (seen.code == kStatusIndexOutOfRange)
    return fail(ETC_EXECUTION, "quantized_embedding: index " + std::to_string(seen.value) + " is outside 0.." + std::to_string(seen.bound));
  if (seen.code == kStatusNonFiniteLogit)
    return fail(ETC_EXECUTION, "sample: logit " + std::to_string(seen.value) + " is not finite");
  if (seen.code == 3) return fail(ETC_EXECUTION, "quantized_linear: a pipeline wait inside the kernel ran out; the launch gave up");
  if (seen.code == 4) return fail(ETC_EXECUTION, "tensor parallel: a peer never arrived at the all-reduce; the launch gave up");
  return fail(ETC_EXECUTION, "device reported status " + std::to_string(seen.code));
}

extern "C" {

const char* etc_last_error_message(void) { return last_error().c_str(); }
const char* etc_version(void) { return "effect-torch-b200 0.1 (sm_100a)"; }

etc_status etc_device_count(int* out_count) {
  if (!out_count) return fail(ETC_INVALID_ARGUMENT, "out_count is null");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  *out_count = n;
  return ETC_OK;
}

etc_status etc_runtime_create(int device_ordinal, etc_runtime** out) {
  static std::atomic<uint64_t> next_id{1};
  if (!out) return fail(ETC_INVALID_ARGUMENT, "out is null");
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    cudaGetLastError();
    return fail(ETC_UNAVAILABLE, "no CUDA device is available (the cuda backend has no CPU fallback)");
  }
  if (device_ordinal < 0 || device_ordinal >= n)
    return fail(ETC_UNAVAILABLE, "cuda device " + std::to_string(device_ordinal) + " does not exist (" + std::to_string(n) + " present)");
  cudaError_t e = cudaSetDevice(device_ordinal);
  if (e != cudaSuccess) return fail(ETC_UNAVAILABLE, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  cudaDeviceProp prop;
  ETC_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major < 10)
    return fail(ETC_UNAVAILABLE, std::string("device ") + prop.name + " is compute capability " + std::to_string(prop.major) + "." +
                                     std::to_string(prop.minor) + "; this backend is built for sm_100a only");
  etc_runtime* rt = new etc_runtime();
  rt->id = next_id++;
  rt->device = device_ordinal;
  rt->sm_count = prop.multiProcessorCount;
  e = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc((void**)&rt->d_status, sizeof(DeviceStatus));
  if (e == cudaSuccess) e = cudaMemset(rt->d_status, 0, sizeof(DeviceStatus));
  if (e == cudaSuccess) e = cudaMallocHost((void**)&rt->h_status, sizeof(DeviceStatus));
  if (e == cudaSuccess) e = cudaMalloc((void**)&rt->d_sampled, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMallocHost((void**)&rt->h_sampled, sizeof(uint32_t));
  // reserve the fixed scratch array of the allocation-free linear now, not inside its first call
  if (e == cudaSuccess) e = static_scratch_prepare(device_ordinal);
  if (e != cudaSuccess) {
    delete rt;
    return fail(ETC_UNAVAILABLE, std::string("runtime setup failed: ") + cudaGetErrorString(e));
  }
  std::memset(rt->h_status, 0, sizeof(DeviceStatus));
  *out = rt;
  return ETC_OK;
}

etc_status etc_runtime_capabilities(etc_runtime* rt, etc_capabilities* out) {
  ETC_TRY(activate(rt));
  if (!out) return fail(ETC_INVALID_ARGUMENT, "out is null");
  cudaDeviceProp prop;
  ETC_CUDA(cudaGetDeviceProperties(&prop, rt->device));
  std::memset(out, 0, sizeof(*out));
  // f64 appears inside kernels (norms, rotary angles, the exact attention) but is not a tensor dtype of this backend
  out->dtype_mask = (1u << ETC_DTYPE_F32) | (1u << ETC_DTYPE_F16) | (1u << ETC_DTYPE_BF16) | (1u << ETC_DTYPE_U8) |
                    (1u << ETC_DTYPE_U32) | (1u << ETC_DTYPE_I64);
  out->feature_mask = 0x3u;  // compilation (the decoder plan) and asynchronous execution (stream launches)
  out->device_ordinal = rt->device;
  out->sm_count = rt->sm_count;
  out->compute_major = prop.major;
  out->compute_minor = prop.minor;
  out->device_memory_bytes = (uint64_t)prop.totalGlobalMem;
  std::strncpy(out->device_name, prop.name, sizeof(out->device_name) - 1);
  return ETC_OK;
}

etc_status etc_runtime_destroy(etc_runtime* rt) {
  if (!valid(rt)) return fail(ETC_INVALID_HANDLE, "runtime handle is invalid or already destroyed");
  cudaSetDevice(rt->device);
  cudaStreamSynchronize(rt->stream);
  for (auto& kv : rt->allocations) cudaFree(kv.first);
  rt->allocations.clear();
  cudaFree(rt->d_status);
  cudaFreeHost(rt->h_status);
  cudaFree(rt->d_sampled);
  cudaFreeHost(rt->h_sampled);
  cudaStreamDestroy(rt->stream);
  rt->magic = 0;
  delete rt;
  return ETC_OK;
}

etc_status etc_runtime_stream(etc_runtime* rt, void** out_stream) {
  if (!valid(rt)) return fail(ETC_INVALID_HANDLE, "runtime handle is invalid");
  *out_stream = (void*)rt->stream;
  return ETC_OK;
}

etc_status etc_runtime_synchronize(etc_runtime* rt) {
  ETC_TRY(activate(rt));
  return rt->check_status();
}

etc_status etc_runtime_launch_count(etc_runtime* rt, uint64_t* out) {
  if (!valid(rt)) return fail(ETC_INVALID_HANDLE, "runtime handle is invalid");
  *out = rt->launches.load();
  return ETC_OK;
}

etc_status etc_runtime_memory_bytes(etc_runtime* rt, uint64_t* out) {
  if (!valid(rt)) return fail(ETC_INVALID_HANDLE, "runtime handle is invalid");
  *out = rt->memory_bytes.load();
  return ETC_OK;
}

etc_status etc_alloc(etc_runtime* rt, size_t bytes, void** out_d_ptr) {
  ETC_TRY(activate(rt));
  if (!out_d_ptr) return fail(ETC_INVALID_ARGUMENT, "out pointer is null");
  return rt->device_alloc(bytes, out_d_ptr);
}

etc_status etc_free(etc_runtime* rt, void* d_ptr) {
  ETC_TRY(activate(rt));
  ETC_CUDA(cudaStreamSynchronize(rt->stream));
  return rt->device_free(d_ptr);
}

etc_status etc_upload(etc_runtime* rt, void* d_dst, const void* h_src, size_t bytes) {
  ETC_TRY(activate(rt));
  if (bytes == 0) return ETC_OK;
  cudaError_t e = cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, rt->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
  if (e != cudaSuccess) return fail(ETC_TRANSFER, std::string("upload failed: ") + cudaGetErrorString(e));
  return ETC_OK;
}

etc_status etc_download(etc_runtime* rt, void* h_dst, const void* d_src, size_t bytes) {
  ETC_TRY(activate(rt));
  if (bytes == 0) return ETC_OK;
  cudaError_t e = cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, rt->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
  if (e != cudaSuccess) return fail(ETC_TRANSFER, std::string("readback failed: ") + cudaGetErrorString(e));
  return ETC_OK;
}

}  // extern "C"
