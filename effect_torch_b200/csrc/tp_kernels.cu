// All-reduce over peer memory for the tensor-parallel decoder: hidden += sum over ranks of every rank's partial sum, and
// the exchange of every rank's best logit for a vocabulary-parallel head.
//
// Every rank owns one exported region (layout: kTp* in kernels.h): three flag arrays (one 32-bit epoch per peer,
// written BY that peer), a table of (best logit, token) pairs, and two exchange buffers that the o and down projections
// alternate between, each an inbox with one slot per sender and a table of totals. Data moves by plain STORES into the
// peers' regions over NVLink (posted writes: no round trip is waited for), followed by a system-wide fence and a store
// of the epoch into the peer's flag array; all reads are local: a warp polls all peers' flags at once with relaxed loads
// and fences once when they have all arrived. Nothing here uses multicast.
//
//   one shot (up to 4 ranks, or forced): every rank stores its whole partial sum into slot `rank` of every rank's inbox; after
//     one flag exchange every rank adds the slots in rank order onto its hidden state. (world - 1) x message bytes leave
//     every rank.
//   two shot (8 ranks, or forced): rank r stores slice q of its partial sum into slot r of rank q's inbox (reduce-scatter); after
//     the first flag exchange rank q adds the slots of its slice in rank order, adds the total onto its own hidden state
//     and stores it into every peer's table of totals (all-gather); after the second exchange every rank adds the other
//     slices' totals onto its hidden state. 2 (world - 1) / world x message bytes leave every rank.
//   Both give bit-identical hidden states on all ranks: the sum over ranks first, in rank order, then onto hidden.
//
// The partial sum is either read from a buffer or, with `sum.splits > 0`, added up from the row-parallel projection's
// split-K partials on the way out, so that projection needs no sum launch of its own. Two buffers suffice: a rank can
// only store for the second next all-reduce after every peer entered the next one, i.e. finished reading this one.
//
// CTAs of one launch never wait for one another: a thread only reads entries of this rank's own slot and of the hidden
// state that it wrote itself, everything else comes from peers and is guarded by their flags; the last CTA to arrive at a
// phase counter publishes this rank's flag. Every wait is bounded by `wait_cycles`: on expiry the kernel records status
// code 4 and returns.
#include <algorithm>

#include <cstdlib>

#include "chain.cuh"
#include "kernels.h"

namespace etc {

namespace {

// data a peer stored into this rank's region: never from a stale L1 line
__device__ __forceinline__ float4 load_inbox4(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_peer4(float4* p, const float4& v) {
  asm volatile("st.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t load_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// All 32 lanes of a CTA's first warp: lane r watches peer r's entry of flag array `which` in this rank's region, all
// peers at once, until every peer has published `epoch`; one system-wide fence then orders the inbox reads that follow
// (relaxed polls + fence instead of one acquire load after another: the cost does not grow with the number of ranks).
__device__ bool wait_for_peers(const PeerView& pv, int which, uint32_t epoch, long long start, long long wait_cycles) {
  const int r = threadIdx.x & 31;
  const bool mine = r < pv.world && r != pv.rank;
  const uint32_t* flag = pv.flags[pv.rank] + which * kTpFlagStride + (mine ? r : pv.rank);
  bool arrived = false;
  for (;;) {
    const bool ready = !mine || (int32_t)(load_relaxed_sys(flag) - epoch) >= 0;
    if (__all_sync(0xffffffffu, ready)) {
      arrived = true;
      break;
    }
    if (__any_sync(0xffffffffu, clock64() - start > wait_cycles)) break;
    __nanosleep(40);
  }
  __threadfence_system();
  __syncwarp();
  return arrived;
}
// First warp of a CTA, after its lane 0 fenced what has to be visible: lane r stores the epoch into peer r's flag array.
__device__ void publish_to_peers(const PeerView& pv, int which, uint32_t epoch) {
  const int r = threadIdx.x & 31;
  __syncwarp();
  if (r < pv.world && r != pv.rank) {
    __threadfence_system();
    store_relaxed_sys(pv.flags[r] + which * kTpFlagStride + pv.rank, epoch);
  }
}
// First warp of a CTA, after a __syncthreads that follows the CTA's stores: lane 0 fences them system-wide and arrives at
// phase counter `bar`; the warp of the last CTA of the grid to arrive publishes flag array `which` to the peers.
__device__ void arrive_and_publish(const PeerView& pv, uint32_t* bar, int which, uint32_t epoch) {
  int last = 0;
  if ((threadIdx.x & 31) == 0) {
    __threadfence_system();
    last = atomicAdd(bar, 1u) == gridDim.x - 1;
    if (last) __threadfence_system();
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (last) publish_to_peers(pv, which, epoch);
}

// ctr: [0] epoch of the last completed all-reduce, [1] CTAs done, [2] / [3] phase arrivals, [4] epoch of the last pick exchange
template <bool TWO_SHOT>
__global__ void __launch_bounds__(256) tp_allreduce_kernel(PeerView pv, int buffer, float* __restrict__ hidden, size_t count4,
                                                           DeferredSum sum, int columns, const float* __restrict__ partial,
                                                           uint32_t* ctr, long long wait_cycles, unsigned long long* status,
                                                           int chain) {
  __shared__ uint32_t epoch_s;
  __shared__ int ok_s;
  if (chain >= 1) chain_release();  // the kernel after this one may be scheduled; it waits for this one to complete
  if (chain >= 2) chain_wait();     // launched under the projection's tail: its partials are complete from here on
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  const long long start = clock64();
  if (threadIdx.x == 0) {
    epoch_s = *reinterpret_cast<volatile uint32_t*>(ctr) + 1;
    ok_s = 1;
  }
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const int world = pv.world, rank = pv.rank;
  const size_t slice = TWO_SHOT ? (count4 + world - 1) / world : count4;  // float4 elements per inbox slot
  float4* h4 = reinterpret_cast<float4*>(hidden);
  const int columns4 = columns / 4;
  // ---- phase A: this rank's partial sum goes out, slice q (two shot) or all of it (one shot) into slot `rank` of rank q
  for (size_t i = tid; i < count4; i += stride) {
    float4 val;
    if (sum.splits > 0) {
      const size_t v = i / columns4, c4 = i - v * columns4;
      val = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < sum.splits; ++s) {
        const float4 p = *reinterpret_cast<const float4*>(sum.partials + ((size_t)s * sum.vpad + v) * sum.rows_padded + 4 * c4);
        val.x += p.x; val.y += p.y; val.z += p.z; val.w += p.w;
      }
    } else {
      val = reinterpret_cast<const float4*>(partial)[i];
    }
    if (TWO_SHOT) {
      const int q = (int)(i / slice);
      store_peer4(reinterpret_cast<float4*>(pv.inbox[q][buffer]) + (size_t)rank * slice + (i - (size_t)q * slice), val);
    } else {
      for (int q = 0; q < world; ++q) store_peer4(reinterpret_cast<float4*>(pv.inbox[q][buffer]) + (size_t)rank * slice + i, val);
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    arrive_and_publish(pv, ctr + 2, 0, epoch);
    // the peers fill the other slots of this rank's inbox; the entries of its own slot that a thread adds up below are
    // the ones that same thread stored above, so CTAs of this grid do not wait for one another
    const bool arrived = wait_for_peers(pv, 0, epoch, start, wait_cycles);
    if (threadIdx.x == 0 && !arrived) ok_s = 0;
  }
  __syncthreads();
  const float4* inbox = reinterpret_cast<const float4*>(pv.inbox[rank][buffer]);
  if (!TWO_SHOT) {
    for (size_t i = tid; i < count4 && ok_s; i += stride) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const float4 p = load_inbox4(inbox + (size_t)r * slice + i);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
      }
      const float4 h = h4[i];
      h4[i] = make_float4(h.x + acc.x, h.y + acc.y, h.z + acc.z, h.w + acc.w);
    }
  } else {
    const size_t lo = slice * rank < count4 ? slice * rank : count4, hi = lo + slice < count4 ? lo + slice : count4;
    // ---- phase B: total of this rank's slice, onto its own hidden state and out to every peer's table of totals
    for (size_t i = tid; i < hi && ok_s; i += stride) {  // the elements of the slice that this thread sent in phase A
      if (i < lo) continue;
      const size_t j = i - lo;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const float4 p = load_inbox4(inbox + (size_t)r * slice + j);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
      }
      const float4 h = h4[lo + j];
      h4[lo + j] = make_float4(h.x + acc.x, h.y + acc.y, h.z + acc.z, h.w + acc.w);
      for (int q = 0; q < world; ++q)
        if (q != rank) store_peer4(reinterpret_cast<float4*>(pv.totals[q][buffer]) + lo + j, acc);
    }
    __syncthreads();
    if (threadIdx.x < 32 && ok_s) {  // ok_s is not written between the barriers around this block's predecessor and here
      arrive_and_publish(pv, ctr + 3, 1, epoch);
      const bool arrived = wait_for_peers(pv, 1, epoch, start, wait_cycles);
      __syncwarp();
      if (threadIdx.x == 0 && !arrived) ok_s = 0;
    }
    __syncthreads();
    // ---- phase C: the other slices' totals onto the hidden state
    const float4* totals = reinterpret_cast<const float4*>(pv.totals[rank][buffer]);
    for (size_t i = tid; i < count4 && ok_s; i += stride) {
      if (i >= lo && i < hi) continue;
      const float4 p = load_inbox4(totals + i);
      const float4 h = h4[i];
      h4[i] = make_float4(h.x + p.x, h.y + p.y, h.z + p.z, h.w + p.w);
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
  if (threadIdx.x < 32) {
    if (threadIdx.x == 0) __threadfence_system();  // the argmax kernel that wrote this rank's pairs finished before this kernel started
    publish_to_peers(pv, 2, epoch);
    const bool arrived = wait_for_peers(pv, 2, epoch, clock64(), wait_cycles);
    if (threadIdx.x == 0) ok_s = arrived ? 1 : 0;
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
                                const float* partial, bool two_shot, uint32_t* counters, long long wait_cycles, int sm_count,
                                DeviceStatus* status, cudaStream_t stream) {
  const size_t count4 = count / 4;
  // every thread has a few 16-byte stores in flight; no more CTAs than SMs, so that all of them are resident
  const unsigned grid = (unsigned)std::min<size_t>((size_t)std::max(1, sm_count), std::max<size_t>(1, (count4 + 1023) / 1024));
  // How the kernel sits in the stream's chain of programmatic launches (ETC_TP_CHAIN overrides, for measurements):
  //   1 (default) launched the ordinary way, after the projection has ended, but it lets the kernel after it be
  //     scheduled at once, so that kernel's launch hides behind the exchange: 16.85 ms per step at 4 ranks;
  //   0 no early scheduling either: 17.0 ms;  2 also launched under the projection's tail: 18.05 ms (measured slower twice).
  static const int chain = [] {
    const char* v = std::getenv("ETC_TP_CHAIN");
    return v ? std::atoi(v) : 1;
  }();
  unsigned long long* code = &status->code;
  if (chain >= 2) {
    if (two_shot) return launch_chained(tp_allreduce_kernel<true>, dim3(grid), dim3(256), 0, stream, view, buffer, hidden, count4, sum, columns, partial, counters, wait_cycles, code, chain);
    return launch_chained(tp_allreduce_kernel<false>, dim3(grid), dim3(256), 0, stream, view, buffer, hidden, count4, sum, columns, partial, counters, wait_cycles, code, chain);
  }
  if (two_shot) tp_allreduce_kernel<true><<<grid, 256, 0, stream>>>(view, buffer, hidden, count4, sum, columns, partial, counters, wait_cycles, code, chain);
  else tp_allreduce_kernel<false><<<grid, 256, 0, stream>>>(view, buffer, hidden, count4, sum, columns, partial, counters, wait_cycles, code, chain);
  return cudaGetLastError();
}

cudaError_t launch_tp_pick(const PeerView& view, int batch, uint32_t* tokens, uint32_t* counters, long long wait_cycles,
                           DeviceStatus* status, cudaStream_t stream) {
  tp_pick_kernel<<<1, 256, 0, stream>>>(view, batch, tokens, counters, wait_cycles, &status->code);
  return cudaGetLastError();
}

}  // namespace etc
