// Measurement program (not part of the library): what one SM of a B200 can retire per cycle on its two tensor paths.
//
//   1. tcgen05.mma alone: cycles per instruction for kind::f16 (K = 16) with the A operand in tensor memory or in shared
//      memory, M in {64, 128}, N in {16 .. 256}, 1 / 2 / 4 independent accumulators; and kind::f8f6f4 (K = 32).
//   2. mma.sync.m16n8k16 (the legacy path) alone: instructions per cycle per SM for 4 / 8 / 16 warps.
//   3. both at once in one CTA: one lane issues tcgen05.mma back to back while W warps run mma.sync; reports the rate of
//      each next to its stand-alone rate, which answers whether the two paths share one pipe.
// Operands are zeros / small constants; only issue and completion times matter. Every wait is bounded and tensor
// memory is always released.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o tensor_issue_probe tensor_issue_probe.cu && ./tensor_issue_probe
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  desc |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  desc |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  desc |= (uint64_t)1 << 46;
  return desc;
}
__device__ __forceinline__ void umma_f16_ts(uint32_t d, uint32_t a, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
               ::"r"(d), "r"(a), "l"(b_desc), "r"(idesc), "r"(acc), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_f16_ss(uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
               ::"r"(d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_f8_ts(uint32_t d, uint32_t a, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
               ::"r"(d), "r"(a), "l"(b_desc), "r"(idesc), "r"(acc), "r"(0u) : "memory");
}
__device__ __forceinline__ void legacy_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// kind 0 = f16 (K 16), 1 = f8f6f4 (K 32, A in tensor memory only). form 0 = A in tensor memory, 1 = A in shared memory.
// `legacy_warps` extra warps run mma.sync while the tcgen05 chain is in flight (0 = tcgen05 alone); `umma_reps` = 0
// runs the legacy warps alone for `legacy_iters` rounds of 8 instructions.
// out[0] issue cycles, out[1] cycles until the commit arrived, out[2] commit seen, out[3] legacy instructions retired by
// the CTA inside the window out[4] (cycles, slowest warp).
__global__ void __launch_bounds__(640) probe(int kind, int form, int M, int N, int naccs, int umma_reps, int legacy_warps,
                                              int legacy_iters, long long* out) {
  extern __shared__ __align__(128) unsigned char smem[];  // 64 KB of zeros: A at 0, B at 8 KB
  __shared__ uint64_t bar;
  __shared__ uint32_t holder;
  __shared__ volatile int stop;
  __shared__ unsigned long long legacy_count;
  __shared__ unsigned long long legacy_cycles;
  for (int i = threadIdx.x; i < 16384; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    stop = 0;
    legacy_count = 0;
    legacy_cycles = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&holder)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tbase = holder;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    if (umma_reps > 0) {
      // instruction descriptor: D = f32 (bit 4), A / B formats 0 (f16 resp. e4m3), N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
      const uint32_t kbytes = 16u;  // one 8-row core matrix row is 16 bytes for both kinds
      const uint64_t a_desc = make_desc(smem_u32(smem), (uint32_t)M * kbytes, 128u);
      const uint64_t b_desc = make_desc(smem_u32(smem + 8192), (uint32_t)N * kbytes, 128u);
      const long long t0 = clock64();
#pragma unroll 8
      for (int r = 0; r < umma_reps; ++r) {
        const uint32_t d = tbase + (uint32_t)((r & (naccs - 1)) * N);  // accumulators at columns [0, naccs * N) <= 256
        const uint32_t a_t = tbase + 256u + (uint32_t)((r & 7) * 8);
        if (kind == 1) umma_f8_ts(d, a_t, b_desc, idesc, r >= naccs);
        else if (form == 0) umma_f16_ts(d, a_t, b_desc, idesc, r >= naccs);
        else umma_f16_ss(d, a_desc, b_desc, idesc, r >= naccs);
      }
      const long long t1 = clock64();
      tc_commit(&bar);
      bool ok = false;
      for (unsigned spin = 0; spin < (1u << 22) && !(ok = mbar_try_wait(&bar, 0)); ++spin) {}
      const long long t2 = clock64();
      stop = 1;
      if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = ok ? 1 : 0; }
    }
  } else if (warp >= 4 && warp < 4 + legacy_warps) {
    uint32_t a[4] = {threadIdx.x, 1u, 2u, 3u};
    float c[8][4] = {};
    unsigned long long done = 0;
    const long long t0 = clock64();
    for (int it = 0; it < legacy_iters && !(umma_reps > 0 && stop); ++it) {
#pragma unroll
      for (int j = 0; j < 8; ++j) legacy_mma(c[j], a, 5u, 7u);
      done += 8;
    }
    const long long t1 = clock64();
    float s = 0.f;
    for (int j = 0; j < 8; ++j) s += c[j][0] + c[j][1] + c[j][2] + c[j][3];
    if (s == 12345.678f) out[7] = 1;
    if ((threadIdx.x & 31) == 0) {
      atomicAdd(&legacy_count, done);
      atomicMax(&legacy_cycles, (unsigned long long)(t1 - t0));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0) { out[3] = (long long)legacy_count; out[4] = (long long)legacy_cycles; }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(512u) : "memory");
  }
}

static bool run(int kind, int form, int M, int N, int naccs, int umma_reps, int legacy_warps, int legacy_iters, long long* d_out,
                long long* h) {
  for (int it = 0; it < 2; ++it) {
    cudaMemset(d_out, 0, 64);
    probe<<<148, 128 + 32 * legacy_warps, 65536>>>(kind, form, M, N, naccs, umma_reps, legacy_warps, legacy_iters, d_out);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      printf("error: %s\n", cudaGetErrorString(e));
      return false;
    }
  }
  cudaMemcpy(h, d_out, 64, cudaMemcpyDeviceToHost);
  return true;
}

int main() {
  long long* d_out;
  cudaMalloc(&d_out, 64);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
  long long h[8];
  const int reps = 512;
  printf("# 1. tcgen05.mma alone, one issuing lane per SM, %d instructions back to back (cycles per instruction: issue / until commit)\n", reps);
  printf("kind form M N accumulators issue_cycles complete_cycles weights_per_cycle_A_side\n");
  for (int form = 0; form < 2; ++form)
    for (int M = 64; M <= 128; M *= 2)
      for (int N = 16; N <= 256; N *= 2)  // M = 128 needs N % 16 == 0
        for (int naccs = 1; naccs <= 4; naccs *= 2) {
          if (naccs * N > 256) continue;
          if (!run(0, form, M, N, naccs, reps, 0, 0, d_out, h)) return 1;
          printf("f16 %s %d %d %d %.1f %.1f %.1f\n", form ? "smem" : "tmem", M, N, naccs, (double)h[0] / reps, (double)h[1] / reps,
                 (double)M * 16 * reps / (double)h[1]);
        }
  for (int N : {32, 96, 256}) {
    if (!run(1, 0, 128, N, 1, reps, 0, 0, d_out, h)) return 1;
    printf("f8f6f4 tmem 128 %d 1 %.1f %.1f %.1f\n", N, (double)h[0] / reps, (double)h[1] / reps, 128.0 * 32 * reps / (double)h[1]);
  }
  printf("# 2. mma.sync.m16n8k16 alone (instructions per cycle per SM; one instruction = 4096 flop)\n");
  printf("warps instructions_per_cycle tflops_at_1965MHz_148SM\n");
  double alone[3] = {0, 0, 0};
  int wi = 0;
  for (int warps : {4, 8, 16}) {
    if (!run(0, 0, 128, 32, 1, 0, warps, 4000, d_out, h)) return 1;
    const double ipc = (double)h[3] / (double)h[4];
    alone[wi++] = ipc;
    printf("%d %.3f %.0f\n", warps, ipc, ipc * 4096 * 1.965e9 * 148 / 1e12);
  }
  printf("# 3. both paths in one CTA: tcgen05 f16 A-in-tmem M=128 (N as given) back to back beside W mma.sync warps\n");
  printf("N legacy_warps umma_complete_cycles legacy_instructions_per_cycle legacy_alone\n");
  wi = 0;
  for (int warps : {4, 8, 16}) {
    for (int N : {32, 256}) {
      if (!run(0, 0, 128, N, 1, 4096, warps, 1 << 20, d_out, h)) return 1;
      printf("%d %d %.1f %.3f %.3f\n", N, warps, (double)h[1] / 4096, (double)h[3] / (double)h[4], alone[wi]);
    }
    ++wi;
  }
  cudaFree(d_out);
  return 0;
}
