// All-reduce over peer memory for the tensor-parallel decoder: hidden += sum over ranks of partial[rank], and the exchange
// of every rank's best logit for a vocabulary-parallel head.
//
// Every rank owns one exported region (layout: tp_region_* in kernels.h): three flag arrays (one 32-bit epoch per peer,
// written BY that peer), a table of (best logit, token) pairs, and two partial-sum buffers that the o and down
// projections alternate between. Ranks read their peers' buffers with plain loads over NVLink; nothing here uses
// multicast. Two buffers suffice: a rank can only reach the second next projection after every peer entered the next
// all-reduce, i.e. finished reading in this one.
//
//   one shot (2 ranks, or small messages): publish "my partial of epoch e is complete" into every peer's flags, wait
//     until all peers have published e, then every CTA adds the partial sums of all ranks in rank order on top of its
//     local hidden state: (world - 1) x message bytes cross NVLink into every rank.
//   two shot (4-8 ranks): rank r first reduces slice r of the message over all ranks (in rank order) and writes the
//     total back into slice r of its own buffer (reduce-scatter); after a second flag exchange every rank adds every
//     slice's total, read from its owner, onto its hidden state (all-gather): 2 (world - 1) / world x message bytes.
//   Both give bit-identical hidden states on all ranks (the same additions in the same order).
//
// With `sum.splits > 0` the kernel first adds up the row-parallel projection's split-K partials into this rank's buffer,
// so that projection needs no sum launch of its own and its result never passes through the hidden state.
//
// CTAs of one launch wait for one another at the phase boundaries; the grid is at most 64 CTAs of 256 threads without
// shared memory, launched after the previous kernel of the stream has ended, so all of them are resident. Every wait is
// bounded by `wait_cycles`: on expiry the kernel records status code 4 and returns.
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
__device__ __forceinline__ uint32_t load_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 load_peer4(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// Thread 0 of a CTA: waits until every peer has published `epoch` into flag array `which` of this rank's region.
__device__ bool wait_for_peers(const PeerView& pv, int which, uint32_t epoch, long long start, long long wait_cycles) {
  for (int r = 0; r < pv.world; ++r) {
    if (r == pv.rank) continue;
    while ((int32_t)(load_acquire_sys(pv.flags[pv.rank] + which * kTpFlagStride + r) - epoch) < 0) {
      if (clock64() - start > wait_cycles) return false;
      __nanosleep(100);
    }
  }
  return true;
}
__device__ void publish_to_peers(const PeerView& pv, int which, uint32_t epoch) {
  for (int r = 0; r < pv.world; ++r)
    if (r != pv.rank) store_release_sys(pv.flags[r] + which * kTpFlagStride + pv.rank, epoch);
}
// Thread 0 of a CTA: arrives at phase counter `bar`; the last CTA of the grid to arrive publishes flag array `which`.
// The CTA's earlier global writes (made visible by the __syncthreads before this call) are fenced system-wide first.
__device__ void arrive_and_publish(const PeerView& pv, uint32_t* bar, int which, uint32_t epoch) {
  __threadfence_system();
  if (atomicAdd(bar, 1u) == gridDim.x - 1) {
    __threadfence_system();
    publish_to_peers(pv, which, epoch);
  }
}
__device__ bool wait_for_grid(const uint32_t* bar, long long start, long long wait_cycles) {
  while (load_acquire_gpu(bar) < gridDim.x) {
    if (clock64() - start > wait_cycles) return false;
    __nanosleep(50);
  }
  return true;
}

// ctr: [0] epoch of the last completed all-reduce, [1] CTAs done, [2] / [3] phase arrivals
template <bool TWO_SHOT>
__global__ void __launch_bounds__(256) tp_allreduce_kernel(PeerView pv, int buffer, float* __restrict__ hidden, size_t count4,
                                                           DeferredSum sum, int columns, uint32_t* ctr, long long wait_cycles,
                                                           unsigned long long* status) {
  __shared__ uint32_t epoch_s;
  __shared__ int ok_s;
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  float4* mine = reinterpret_cast<float4*>(pv.partial[pv.rank][buffer]);
  const long long start = clock64();
  if (threadIdx.x == 0) {
    epoch_s = *reinterpret_cast<volatile uint32_t*>(ctr) + 1;
    ok_s = 1;
  }
  __syncthreads();
  const uint32_t epoch = epoch_s;
  // ---- phase 0: this rank's partial sum is complete in its buffer, tell the peers
  if (sum.splits > 0) {
    const int columns4 = columns / 4;
    for (size_t i = tid; i < count4; i += stride) {
      const size_t v = i / columns4, c4 = i - v * columns4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < sum.splits; ++s) {
        const float4 p = *reinterpret_cast<const float4*>(sum.partials + ((size_t)s * sum.vpad + v) * sum.rows_padded + 4 * c4);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
      }
      mine[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      arrive_and_publish(pv, ctr + 2, 0, epoch);
      if (TWO_SHOT && !wait_for_grid(ctr + 2, start, wait_cycles)) ok_s = 0;  // slice `rank` below spans other CTAs' sums
    }
  } else if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();  // the projection that filled this rank's buffer finished before this kernel started
    publish_to_peers(pv, 0, epoch);
  }
  if (threadIdx.x == 0 && ok_s && !wait_for_peers(pv, 0, epoch, start, wait_cycles)) ok_s = 0;
  __syncthreads();
  float4* h4 = reinterpret_cast<float4*>(hidden);
  if (!TWO_SHOT) {
    if (ok_s) {
      if (sum.splits > 0 && threadIdx.x == 0 && !wait_for_grid(ctr + 2, start, wait_cycles)) ok_s = 0;
      __syncthreads();
      for (size_t i = tid; i < count4 && ok_s; i += stride) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);  // the ranks' sum first, then onto hidden: what the two-shot form computes
        for (int r = 0; r < pv.world; ++r) {
          const float4 p = load_peer4(reinterpret_cast<const float4*>(pv.partial[r][buffer]) + i);
          acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        const float4 h = h4[i];
        h4[i] = make_float4(h.x + acc.x, h.y + acc.y, h.z + acc.z, h.w + acc.w);
      }
    }
  } else {
    const size_t slice = (count4 + pv.world - 1) / pv.world;
    if (ok_s) {
      // ---- phase 1: total of this rank's slice over all ranks, written back into this rank's buffer
      const size_t lo = slice * pv.rank < count4 ? slice * pv.rank : count4, hi = lo + slice < count4 ? lo + slice : count4;
      for (size_t i = lo + tid; i < hi; i += stride) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < pv.world; ++r) {
          const float4 p = load_peer4(reinterpret_cast<const float4*>(pv.partial[r][buffer]) + i);
          acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        mine[i] = acc;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && ok_s) {
      arrive_and_publish(pv, ctr + 3, 1, epoch);
      if (!wait_for_grid(ctr + 3, start, wait_cycles) || !wait_for_peers(pv, 1, epoch, start, wait_cycles)) ok_s = 0;
    }
    __syncthreads();
    if (ok_s) {
      // ---- phase 2: every slice's total, read from its owner, onto the hidden state
      for (size_t i = tid; i < count4; i += stride) {
        const int owner = (int)(i / slice);
        const float4 p = load_peer4(reinterpret_cast<const float4*>(pv.partial[owner][buffer]) + i);
        float4 acc = h4[i];
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        h4[i] = acc;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok_s) atomicCAS(status, 0ull, 4ull);  // a peer never arrived
    __threadfence();
    if (atomicAdd(ctr + 1, 1u) == gridDim.x - 1) {  // every CTA is through: reset the phase counters, advance the epoch
      ctr[1] = 0;
      ctr[2] = 0;
      ctr[3] = 0;
      __threadfence();
      ctr[0] = epoch;
    }
  }
}

// One CTA: publishes this rank's (best logit, token) pairs, waits for the peers', keeps per lane the largest logit and
// on ties the lowest token index (crates/runtime/src/sampling.rs:88-105 scans ascending with a strict comparison).
// ctr[4]: epoch of the last exchange.
__global__ void __launch_bounds__(256) tp_pick_kernel(PeerView pv, int batch, uint32_t* __restrict__ tokens, uint32_t* ctr,
                                                      long long wait_cycles, unsigned long long* status) {
  __shared__ int ok_s;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ctr + 4) + 1;
  if (threadIdx.x == 0) {
    __threadfence_system();  // the argmax kernel that wrote this rank's pairs finished before this kernel started
    publish_to_peers(pv, 2, epoch);
    ok_s = wait_for_peers(pv, 2, epoch, clock64(), wait_cycles) ? 1 : 0;
  }
  __syncthreads();
  if (ok_s) {
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
      float best = -INFINITY;
      uint32_t arg = 0xffffffffu;
      for (int r = 0; r < pv.world; ++r) {
        uint2 pick;
        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(pick.x), "=r"(pick.y) : "l"(pv.picks[r] + b) : "memory");
        const float v = __uint_as_float(pick.x);
        if (v > best || (v == best && pick.y < arg)) { best = v; arg = pick.y; }
      }
      tokens[b] = arg == 0xffffffffu ? 0u : arg;
    }
  } else if (threadIdx.x == 0) {
    atomicCAS(status, 0ull, 4ull);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    ctr[4] = epoch;
  }
}

}  // namespace

cudaError_t launch_tp_allreduce(const PeerView& view, int buffer, float* hidden, size_t count, int columns, const DeferredSum& sum,
                                bool two_shot, uint32_t* counters, long long wait_cycles, DeviceStatus* status, cudaStream_t stream) {
  const size_t count4 = count / 4;
  const unsigned grid = (unsigned)std::min<size_t>(64, std::max<size_t>(1, (count4 + 255) / 256));
  if (two_shot)
    tp_allreduce_kernel<true><<<grid, 256, 0, stream>>>(view, buffer, hidden, count4, sum, columns, counters, wait_cycles, &status->code);
  else
    tp_allreduce_kernel<false><<<grid, 256, 0, stream>>>(view, buffer, hidden, count4, sum, columns, counters, wait_cycles, &status->code);
  return cudaGetLastError();
}

cudaError_t launch_tp_pick(const PeerView& view, int batch, uint32_t* tokens, uint32_t* counters, long long wait_cycles,
                           DeviceStatus* status, cudaStream_t stream) {
  tp_pick_kernel<<<1, 256, 0, stream>>>(view, batch, tokens, counters, wait_cycles, &status->code);
  return cudaGetLastError();
}

}  // namespace etc
