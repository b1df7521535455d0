// Next-token sampling on the device, one CTA per logits row: greedy, temperature softmax, top-k and top-p with the
// splitmix64 draw of crates/runtime/src/sampling.rs:35-42, 80-206.
//
// The reference orders candidates by (value descending, token ascending), keeps the first top_k, turns them into
// weights exp((value - max) / temperature), keeps the smallest prefix whose weight reaches top_p x total, and walks that
// prefix subtracting weights from draw = unit x total until it goes negative. Without top-k and top-p it walks the row in
// token order instead. Here every candidate gets the 52-bit sort key (order-preserving bits of the f32 logit, then the
// inverted token), so "the first n candidates", "the smallest prefix reaching a weight" and "the candidate where the walk
// goes negative" are all the same primitive: a radix select, seven 8-bit digits from the top, over a histogram of counts
// or of weights. No candidate list is stored and nothing is sorted; a pass re-reads the row (L2 resident) and evaluates
// exp only for candidates that still match the digits chosen so far. The token-order walk is a block-wide prefix sum over
// per-thread chunks.
//
// Sums are f64 like the reference's but associated differently (histogram bins, a tree over threads), so a comparison of
// a running sum against the draw or the top-p threshold can come out differently only when the two are within about
// vocab x 2^-52 of each other, relative to the total weight.
#include <algorithm>

#include "chain.cuh"
#include "kernels.h"

namespace etc {

namespace {

constexpr int kSampleThreads = 1024;

struct SampleArgs {
  const float* logits;
  int64_t vocab;
  double temperature, top_p;
  int64_t top_k;  // 0: no limit
  uint64_t seed, counter;
  const uint64_t* seeds;     // optional per-row keys (device); the scalars serve every row otherwise
  const uint64_t* counters;
  uint32_t* tokens;
  DeviceStatus* status;
};

__device__ __forceinline__ double random_unit(uint64_t seed, uint64_t counter) {
  uint64_t value = seed ^ (counter * 0x9e3779b97f4a7c15ull);
  value += 0x9e3779b97f4a7c15ull;
  value = (value ^ (value >> 30)) * 0xbf58476d1ce4e5b9ull;
  value = (value ^ (value >> 27)) * 0x94d049bb133111ebull;
  value ^= value >> 31;
  return (double)(value >> 11) * (1.0 / 9007199254740992.0);
}

// Larger logit -> larger key; among equal logits the lower token has the larger key. Tokens are below 2^20.
__device__ __forceinline__ uint64_t sort_key(float v, uint32_t token) {
  const uint32_t u = __float_as_uint(v);
  const uint32_t ordered = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((uint64_t)ordered << 20) | (uint64_t)(0xFFFFFu - token);
}
__device__ __forceinline__ uint32_t key_token(uint64_t key) { return 0xFFFFFu - (uint32_t)(key & 0xFFFFFu); }

struct Shared {
  double hist[256];
  uint32_t count[256];
  double warp_sum[32];
  unsigned long long warp_key[32];
  double acc;
  int digit;
  int found;
};

__device__ double block_sum(Shared& sh, double v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.warp_sum[threadIdx.x >> 5] = v;
  __syncthreads();
  double total = 0.0;
  for (int w = 0; w < kSampleThreads / 32; ++w) total += sh.warp_sum[w];  // the same order in every thread
  return total;
}
__device__ uint64_t block_min_key(Shared& sh, uint64_t v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const uint64_t o = __shfl_xor_sync(0xffffffffu, v, off);
    v = o < v ? o : v;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.warp_key[threadIdx.x >> 5] = v;
  __syncthreads();
  uint64_t best = ~0ull;
  for (int w = 0; w < kSampleThreads / 32; ++w) best = sh.warp_key[w] < best ? sh.warp_key[w] : best;
  return best;
}

enum Crossing { kReaches = 0, kExceeds = 1 };  // running >= target (counts, top-p) or running > target (the draw)

// Among the candidates with key >= floor_key, in descending key order: the first one at which the running sum of
// weights (including its own) reaches / exceeds `target`. Returns its key and, in *before, the sum of all candidates
// ahead of it; found == false when the whole set stays below the target.
template <typename Weight>
__device__ uint64_t radix_select(Shared& sh, const float* x, int64_t vocab, uint64_t floor_key, double target, Crossing crossing,
                                 Weight weight, double* before, bool* found) {
  uint64_t prefix = 0, mask = 0;
  double acc = 0.0;
  bool ok = true;
  for (int pass = 0; pass < 7 && ok; ++pass) {
    const int shift = 48 - 8 * pass;
    __syncthreads();
    if (threadIdx.x < 256) {
      sh.hist[threadIdx.x] = 0.0;
      sh.count[threadIdx.x] = 0u;
    }
    __syncthreads();
    for (int64_t i = threadIdx.x; i < vocab; i += kSampleThreads) {
      const float v = x[i];
      const uint64_t key = sort_key(v, (uint32_t)i);
      if (key < floor_key || (key & mask) != prefix) continue;
      const int bin = (int)((key >> shift) & 255u);
      atomicAdd(&sh.hist[bin], weight(v));
      atomicAdd(&sh.count[bin], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double running = acc;
      int digit = -1;
      for (int b = 255; b >= 0; --b) {
        if (sh.count[b] == 0u) continue;
        const double next = running + sh.hist[b];
        if (crossing == kReaches ? next >= target : next > target) {
          digit = b;
          break;
        }
        running = next;
      }
      sh.digit = digit;
      sh.acc = running;
    }
    __syncthreads();
    if (sh.digit < 0) {
      ok = false;
    } else {
      acc = sh.acc;
      prefix |= (uint64_t)sh.digit << shift;
      mask |= 255ull << shift;
    }
  }
  *before = acc;
  *found = ok;
  return prefix;
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(SampleArgs a) {
  __shared__ Shared sh;
  const int row = blockIdx.x;
  const float* x = a.logits + (int64_t)row * a.vocab;
  const int64_t V = a.vocab;
  // ---- every logit must be finite; the largest one anchors the exponentials
  float best = -INFINITY;
  long long bad = 0x7fffffffffffffffll;
  for (int64_t i = threadIdx.x; i < V; i += kSampleThreads) {
    const float v = x[i];
    if (!isfinite(v)) bad = min(bad, (long long)i);
    best = fmaxf(best, v);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, off));
    bad = min(bad, __shfl_xor_sync(0xffffffffu, bad, off));
  }
  if ((threadIdx.x & 31) == 0) {
    sh.warp_sum[threadIdx.x >> 5] = (double)best;
    sh.warp_key[threadIdx.x >> 5] = (unsigned long long)bad;
  }
  __syncthreads();
  double mx = -INFINITY;
  long long first_bad = 0x7fffffffffffffffll;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    mx = fmax(mx, sh.warp_sum[w]);
    first_bad = min(first_bad, (long long)sh.warp_key[w]);
  }
  if (first_bad != 0x7fffffffffffffffll) {
    if (threadIdx.x == 0) {
      a.tokens[row] = 0u;
      if (atomicCAS(&a.status->code, kStatusNone, kStatusNonFiniteLogit) == kStatusNone) {
        a.status->value = first_bad;
        a.status->bound = V;
      }
    }
    return;
  }
  const double temperature = a.temperature;
  auto weight = [mx, temperature](float v) { return exp(((double)v - mx) / temperature); };
  const double unit = random_unit(a.seeds ? a.seeds[row] : a.seed, a.counters ? a.counters[row] : a.counter);
  const bool has_top_k = a.top_k > 0 && a.top_k < V;

  if (!has_top_k && a.top_p >= 1.0) {
    // ---- walk in token order: per-thread chunks, exclusive prefix over the threads, then the chunk that holds the draw
    const int64_t chunk = (V + kSampleThreads - 1) / kSampleThreads;
    const int64_t lo = min(V, (int64_t)threadIdx.x * chunk), hi = min(V, lo + chunk);
    double mine = 0.0;
    for (int64_t i = lo; i < hi; ++i) mine += weight(x[i]);
    // inclusive scan inside the warp, then over the warps
    double scan = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const double o = __shfl_up_sync(0xffffffffu, scan, off);
      if ((threadIdx.x & 31) >= off) scan += o;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 31) sh.warp_sum[threadIdx.x >> 5] = scan;
    if (threadIdx.x == 0) sh.found = 0;
    __syncthreads();
    double ahead = 0.0, total = 0.0;
    for (int w = 0; w < kSampleThreads / 32; ++w) {
      if (w < (int)(threadIdx.x >> 5)) ahead += sh.warp_sum[w];
      total += sh.warp_sum[w];
    }
    const double exclusive = ahead + scan - mine;
    const double draw = unit * total;
    if (lo < hi && exclusive <= draw && draw < exclusive + mine) {
      double left = draw - exclusive;
      int64_t token = hi - 1;
      for (int64_t i = lo; i < hi; ++i) {
        left -= weight(x[i]);
        if (left < 0.0) {
          token = i;
          break;
        }
      }
      a.tokens[row] = (uint32_t)token;
      sh.found = 1;
    }
    __syncthreads();
    if (threadIdx.x == 0 && !sh.found) a.tokens[row] = (uint32_t)(V - 1);
    return;
  }

  // ---- filtered: candidates in (value descending, token ascending) order
  uint64_t floor_key = 0;  // the retained set is {key >= floor_key}
  double before;
  bool found;
  if (has_top_k) {
    auto one = [](float) { return 1.0; };
    floor_key = radix_select(sh, x, V, 0, (double)a.top_k, kReaches, one, &before, &found);  // the top_k-th candidate: always found
  }
  double mine = 0.0;
  for (int64_t i = threadIdx.x; i < V; i += kSampleThreads)
    if (sort_key(x[i], (uint32_t)i) >= floor_key) mine += weight(x[i]);
  double total = block_sum(sh, mine);
  if (a.top_p < 1.0) {
    const uint64_t last = radix_select(sh, x, V, floor_key, a.top_p * total, kReaches, weight, &before, &found);
    if (found) {  // the prefix ends at this candidate; otherwise every candidate stays
      floor_key = last;
      total = before + weight(x[key_token(last)]);
    }
  }
  const uint64_t picked = radix_select(sh, x, V, floor_key, unit * total, kExceeds, weight, &before, &found);
  uint32_t token;
  if (found) {
    token = key_token(picked);
  } else {  // the walk never went negative: the last retained candidate
    uint64_t lowest = ~0ull;
    for (int64_t i = threadIdx.x; i < V; i += kSampleThreads) {
      const uint64_t key = sort_key(x[i], (uint32_t)i);
      if (key >= floor_key && key < lowest) lowest = key;
    }
    token = key_token(block_min_key(sh, lowest));
  }
  if (threadIdx.x == 0) a.tokens[row] = token;
}

}  // namespace

cudaError_t launch_sample_rows(const float* logits, int64_t rows, int64_t vocab, double temperature, int64_t top_k, double top_p,
                               uint64_t seed, uint64_t counter, const uint64_t* seeds, const uint64_t* counters, uint32_t* tokens,
                               DeviceStatus* status, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  SampleArgs a{logits, vocab, temperature, top_p, top_k, seed, counter, seeds, counters, tokens, status};
  sample_rows_kernel<<<(unsigned)rows, kSampleThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace etc
