// Retained (constant) weights of the C ABI.
#pragma once

#include "common.h"
#include "kernels.h"

struct etc_qweight {
  uint32_t magic = etc::kWeightMagic;
  etc_runtime* rt = nullptr;
  etc::TiledWeight tiled;
};

namespace etc {
etc_status build_qweight(etc_runtime* rt, int codec, const void* const* parts, const int64_t* part_rows, int n_parts,
                         int64_t columns, int interleave8, int on_device, etc_qweight** out, const int* part_codecs = nullptr);
void destroy_qweight(etc_qweight* w);
// Loads the device module that holds the fixed scratch array of etc_qlinear_tiled_static_into and resolves the array's
// address on the current device (static_scratch.cu); this is when the driver reserves the array's 16 MiB.
cudaError_t static_scratch_prepare(int device);
etc_status make_inv_freq(etc_runtime* rt, double theta, int head_dim, double** out_device);
etc_status sample_logits_host(const float* logits, int64_t length, double temperature, int64_t top_k, double top_p,
                              uint64_t seed, uint64_t counter, uint32_t* out_token);
}  // namespace etc
