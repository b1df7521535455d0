// One-shot all-reduce over peer memory for the tensor-parallel decoder: hidden += sum over ranks of partial[rank].
//
// Every rank owns one exported region: a flag array (one 32-bit epoch per peer, written BY that peer), and two
// partial-sum buffers that the o and down projections alternate between. The kernel publishes "my partial of epoch e
// is complete" into every peer's flag array, waits until all peers have published e into its own, then every CTA adds
// the partial sums of all ranks in rank order (so all ranks compute bit-identical results) reading the peers' buffers
// with plain loads over NVLink, on top of its local hidden state. Two buffers suffice: a rank can only reach the
// second next projection after every peer entered the next all-reduce, i.e. finished reading in this one.
// The wait is bounded (about a second): on expiry the kernel records status code 4 and returns.
#include <algorithm>

#include "kernels.h"

namespace etc {

namespace {

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 load_peer4(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) tp_allreduce_kernel(PeerView pv, int buffer, float* __restrict__ hidden, size_t count4,
                                                           uint32_t* epoch_counter, uint32_t* done_counter,
                                                           unsigned long long* status) {
  __shared__ uint32_t epoch_s;
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_counter) + 1;
    if (blockIdx.x == 0) {
      // the projection that filled this rank's partial buffer finished before this kernel started
      __threadfence_system();
      for (int r = 0; r < pv.world; ++r)
        if (r != pv.rank) store_release_sys(pv.flags[r] + pv.rank, epoch);
    }
    bool ok = true;
    const long long start = clock64();
    for (int r = 0; r < pv.world && ok; ++r) {
      if (r == pv.rank) continue;
      while ((int32_t)(load_acquire_sys(pv.flags[pv.rank] + r) - epoch) < 0) {
        if (clock64() - start > (1ll << 31)) { ok = false; break; }
        __nanosleep(100);
      }
    }
    epoch_s = epoch;
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (ok_s) {
    float4* h4 = reinterpret_cast<float4*>(hidden);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count4; i += (size_t)gridDim.x * blockDim.x) {
      float4 acc = h4[i];
      for (int r = 0; r < pv.world; ++r) {
        const float4 p = load_peer4(reinterpret_cast<const float4*>(pv.partial[r][buffer]) + i);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
      }
      h4[i] = acc;
    }
  } else if (threadIdx.x == 0) {
    atomicCAS(status, 0ull, 4ull);  // a peer never arrived
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {  // every CTA has read the epoch: advance it for the next call
      *done_counter = 0;
      __threadfence();
      *epoch_counter = epoch_s;
    }
  }
}

}  // namespace

cudaError_t launch_tp_allreduce(const PeerView& view, int buffer, float* hidden, size_t count, uint32_t* epoch_counter,
                                uint32_t* done_counter, DeviceStatus* status, cudaStream_t stream) {
  const size_t count4 = count / 4;
  const unsigned grid = (unsigned)std::min<size_t>(64, std::max<size_t>(1, (count4 + 255) / 256));
  tp_allreduce_kernel<<<grid, 256, 0, stream>>>(view, buffer, hidden, count4, epoch_counter, done_counter, &status->code);
  return cudaGetLastError();
}

}  // namespace etc
