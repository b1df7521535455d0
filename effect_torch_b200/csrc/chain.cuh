// Programmatic dependent launch for the kernels of a decode step. A kernel launched with launch_chained may be
// scheduled while its predecessor in the stream is still running (as soon as every CTA of the predecessor has called
// chain_release or exited), which hides launch latency and CTA ramp-up between the ~350 short kernels of a step. Such a
// kernel calls chain_wait() before its first access to global memory that an earlier kernel writes or still reads:
// the wait returns once the predecessor has completed and its writes are visible, so the stream's semantics stay
// those of plain serialisation. Both calls do nothing in a kernel that was launched the ordinary way.
#pragma once

#include <cuda_runtime.h>

#include <mutex>
#include <set>
#include <utility>

namespace etc {

__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

// Opts a kernel in to `bytes` of dynamic shared memory once per (kernel, device): the attribute belongs to the function
// on a device, so a process that drives several GPUs has to set it on each. Thread-safe.
template <typename Kernel>
inline cudaError_t opt_in_shared_memory(Kernel kernel, size_t bytes) {
  static std::mutex mutex;
  static std::set<std::pair<const void*, int>> configured;  // kernels of one signature share this instantiation
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  const std::pair<const void*, int> key(reinterpret_cast<const void*>(kernel), device);
  std::lock_guard<std::mutex> lock(mutex);
  if (configured.count(key)) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) configured.insert(key);
  return e;
}

}  // namespace etc
