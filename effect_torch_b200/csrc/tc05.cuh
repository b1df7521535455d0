// Inline-PTX helpers for the tcgen05 kernels: mbarriers with bounded waits, bulk copies, tensor-memory
// allocation / loads / stores, MMA issue and commit, shared-memory matrix descriptors, and the f16 expansion of
// packed Q4_0 / Q8_0 words. Everything here is sm_100a only.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>

namespace etc {
namespace tc05 {

constexpr unsigned kSpinLimit = 1u << 24;  // bounded mbarrier waits (a stage takes microseconds)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// try_wait that lets the hardware park the thread until the phase completes or `hint_ns` passes. Without the hint a
// failed try_wait returns within a few cycles and a polling loop eats the issue slots of the warps that do the work.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns) : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and raises the abort flag) when the phase does not complete within about two
// seconds or kSpinLimit polls, whichever comes first.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
  const long long start = clock64();
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > (1ll << 32)) break;
  }
  *abort_flag = 1;
  return false;
}

// The same for a whole warp: every lane gets the same answer, so the warp can keep using __syncwarp afterwards even
// when the wait gave up on some lanes only.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
}

// Bounded wait for roles with slack (they run stages ahead, or wait for a whole range): poll, then sleep. A sleeping
// warp costs the warps that share its scheduler nothing, unlike a spinning or a parked one.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned sleep_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > (1ll << 32)) break;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
      "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem desc]; accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; LBO = byte distance
// between the two 8-column halves of a K=16 slice, SBO = byte distance between 8-row groups.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  desc |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  desc |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  desc |= (uint64_t)1 << 46;  // descriptor version for sm_100
  return desc;                // base offset 0, layout type 0 (no swizzle)
}

__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// One packed u32 = 8 nibbles, logical column j of the word at bit {0,16,8,24,4,20,12,28}[j] -> four half2
// in column order (c0,c1)(c2,c3)(c4,c5)(c6,c7), times the block scale.
__device__ __forceinline__ void expand_q4(uint32_t q, __half2 scale, uint32_t* out4) {
  const uint32_t magic = 0x64006400u;
  const uint32_t qs = q >> 8;
  const __half2 bias_lo = __floats2half2_rn(1032.0f, 1032.0f);
  const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 bias_hi = __floats2half2_rn(-72.0f, -72.0f);
  out4[0] = h2u(__hmul2(__hsub2(u2h((q & 0x000F000Fu) | magic), bias_lo), scale));
  out4[1] = h2u(__hmul2(__hsub2(u2h((qs & 0x000F000Fu) | magic), bias_lo), scale));
  out4[2] = h2u(__hmul2(__hfma2(u2h((q & 0x00F000F0u) | magic), sixteenth, bias_hi), scale));
  out4[3] = h2u(__hmul2(__hfma2(u2h((qs & 0x00F000F0u) | magic), sixteenth, bias_hi), scale));
}
// Four int8 -> (b0,b1)(b2,b3) times scale.
__device__ __forceinline__ void expand_q8(uint32_t w, __half2 scale, uint32_t* out2) {
  const uint32_t x = w ^ 0x80808080u;
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
  out2[0] = h2u(__hmul2(__hsub2(u2h(__byte_perm(x, 0x64646464u, 0x4140)), bias), scale));
  out2[1] = h2u(__hmul2(__hsub2(u2h(__byte_perm(x, 0x64646464u, 0x4342)), bias), scale));
}

// Q4_K block re-cut to 32 values: code * scale - min (scale = d * sc, min = dmin * m, both rounded to f16 at load).
__device__ __forceinline__ void expand_q4k(uint32_t q, __half2 scale, __half2 neg_min, uint32_t* out4) {
  const uint32_t magic = 0x64006400u;
  const uint32_t qs = q >> 8;
  const __half2 bias_lo = __floats2half2_rn(1024.0f, 1024.0f);
  const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 bias_hi = __floats2half2_rn(-64.0f, -64.0f);
  out4[0] = h2u(__hfma2(__hsub2(u2h((q & 0x000F000Fu) | magic), bias_lo), scale, neg_min));
  out4[1] = h2u(__hfma2(__hsub2(u2h((qs & 0x000F000Fu) | magic), bias_lo), scale, neg_min));
  out4[2] = h2u(__hfma2(__hfma2(u2h((q & 0x00F000F0u) | magic), sixteenth, bias_hi), scale, neg_min));
  out4[3] = h2u(__hfma2(__hfma2(u2h((qs & 0x00F000F0u) | magic), sixteenth, bias_hi), scale, neg_min));
}

// Q5_K block re-cut to 32 int8 codes: code * scale - min.
__device__ __forceinline__ void expand_q8k(uint32_t w, __half2 scale, __half2 neg_min, uint32_t* out2) {
  const uint32_t x = w ^ 0x80808080u;
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
  out2[0] = h2u(__hfma2(__hsub2(u2h(__byte_perm(x, 0x64646464u, 0x4140)), bias), scale, neg_min));
  out2[1] = h2u(__hfma2(__hsub2(u2h(__byte_perm(x, 0x64646464u, 0x4342)), bias), scale, neg_min));
}

__device__ __forceinline__ float silu_tanh(float x) { return x * (tanhf(x * 0.5f) * 0.5f + 0.5f); }

// D[tmem] (+)= A[smem desc] * B[smem desc].
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Makes this thread's earlier generic-proxy writes to shared memory visible to the async proxy (tensor core reads).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace tc05
}  // namespace etc
