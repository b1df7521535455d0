// Tiled linear whose split-K scratch lives in a fixed device array of this library instead of in memory that the
// caller or the runtime allocates. The entry point below performs no device or host allocation at all: it suits
// callers that must not allocate while they run (a step that is replayed inside a latency budget, a host that
// has already handed all device memory to its own pools, a callback in which the allocator may not be entered).
//
// The array is shared by every call in the process that targets the same device, so two calls that overlap in
// time (different streams, different threads) race on it; callers serialise them. Nothing in the array has to be
// zero when a call starts: the linear writes every partial sum and every converted activation it later reads.
//
// When the 16 MiB are taken: the array belongs to this translation unit's device module, which the CUDA runtime
// loads lazily. Looking up the array's device address loads the module, and that is the moment the driver reserves
// the memory on the current device. etc_runtime_create therefore calls static_scratch_prepare, so the reservation
// happens while the runtime is being created, before a host divides the remaining device memory among its own
// pools, and can fail there with a clear error instead of inside the first allocation-free call.
#include <mutex>

#include <algorithm>
#include "kernels.h"
#include "weights.h"

namespace {

constexpr size_t kStaticScratchBytes = (size_t)16 << 20;  // 16 MiB: the stated maximum of etc_qlinear_tiled_static_into
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// Resolves the array's device address for the CURRENT device, once per device.
cudaError_t static_scratch_for_device(int device, void** out) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[device]) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_address[device] = ptr;
  }
  *out = g_scratch_address[device];
  return cudaSuccess;
}

}  // namespace

namespace etc {
// Set-up step, once per device, with that device current (called by etc_runtime_create).
cudaError_t static_scratch_prepare(int device) {
  if (device < 0 || device >= kMaxDevices) return cudaSuccess;  // the entry point itself refuses such ordinals
  void* ignored = nullptr;
  return static_scratch_for_device(device, &ignored);
}
}  // namespace etc

extern "C" {

etc_status etc_qlinear_tiled_static_max_bytes(size_t* max_bytes) {
  if (!max_bytes) return etc::fail(ETC_INVALID_ARGUMENT, "quantized_linear: max_bytes is null");
  *max_bytes = kStaticScratchBytes;
  return ETC_OK;
}

etc_status etc_qlinear_tiled_static_into(etc_runtime* rt, const etc_qweight* w, const float* d_x, int64_t vectors,
                                         const float* d_bias, const float* d_residual, etc_epilogue epilogue,
                                         float* d_out) {
  using namespace etc;
  ETC_TRY(activate(rt));
  if (!w || w->magic != kWeightMagic || w->rt != rt)
    return fail(ETC_INVALID_HANDLE, "weight handle is invalid or belongs to a different runtime");
  if (rt->device < 0 || rt->device >= kMaxDevices)
    return fail(ETC_UNSUPPORTED, "quantized_linear: device ordinal " + std::to_string(rt->device) + " is beyond the static scratch table");
  if (epilogue == ETC_EPILOGUE_SWIGLU && !w->tiled.interleave8)
    return fail(ETC_UNSUPPORTED, "quantized_linear: the swiglu epilogue needs a weight built with interleave8");
  if (epilogue == ETC_EPILOGUE_RESIDUAL && !d_residual)
    return fail(ETC_INVALID_ARGUMENT, "quantized_linear: the residual epilogue needs a residual input");
  if (vectors <= 0) return ETC_OK;
  // the whole call in one pass when its scratch fits; otherwise 256 vectors at a time (a slice needs an eighth or so of
  // what the one-pass plan of a long call needs), and only a slice that does not fit is refused
  const int64_t slice = tiled_scratch_bytes(w->tiled, vectors, rt->sm_count) <= kStaticScratchBytes ? vectors : 256;
  for (int64_t v0 = 0; v0 < vectors; v0 += slice) {
    const size_t need = tiled_scratch_bytes(w->tiled, std::min(slice, vectors - v0), rt->sm_count);
    if (need > kStaticScratchBytes)
      return fail(ETC_INVALID_ARGUMENT, "quantized_linear: this call needs " + std::to_string(need) +
                                            " bytes of scratch, the static scratch holds " + std::to_string(kStaticScratchBytes) +
                                            "; use etc_qlinear_tiled_into with caller scratch");
  }
  void* scratch = nullptr;
  ETC_CUDA(static_scratch_for_device(rt->device, &scratch));
  int launches = 0;
  const int64_t out_cols = epilogue == ETC_EPILOGUE_SWIGLU ? w->tiled.rows / 2 : w->tiled.rows;
  for (int64_t v0 = 0; v0 < vectors; v0 += slice)
    ETC_CUDA(launch_qlinear_tiled(w->tiled, d_x + v0 * w->tiled.columns, std::min(slice, vectors - v0), d_bias,
                                  d_residual ? d_residual + v0 * out_cols : nullptr, epilogue, d_out + v0 * out_cols, scratch, rt->d_status,
                                  rt->sm_count, rt->stream, &launches));
  rt->launches += (uint64_t)launches;
  return ETC_OK;
}

}  // extern "C"
