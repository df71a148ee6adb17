// Inline-PTX wrappers for the Blackwell (sm_100a) tensor-core path: mbarriers, proxy fences,
// tensor-memory (TMEM) allocation, tcgen05.mma / commit / ld, and the shared-memory matrix
// descriptors of the 128-byte-swizzled operand tiles.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mc {
namespace tc {

// Device status word: 0 = ok, otherwise the code of the first bounded wait that ran out
// (kernel id * 16 + role).  Read back by mc_device_status().  File-scope on purpose: this header
// is included by exactly one translation unit (conv_tc.cu), which keeps the build free of
// relocatable device code.
static __device__ int g_status = 0;


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that lets the hardware suspend the thread for up to `hint_ns` while the phase is pending,
// instead of burning issue slots in a polling loop.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait (about one second of SM clock).  Returns false if another role already gave up, or
// if the limit ran out, in which case it raises the abort flag of the block and the status word
// of the device.
// sleep_ns = 0 (the default): loop on mbarrier.try_wait, which suspends the thread in hardware for a
// bounded time slice while the phase is pending and wakes it as soon as the phase completes - the
// right thing for the single threads that hand stages over.  sleep_ns > 0: back off between polls,
// for roles where a whole warp waits for something that is far away.
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int code, unsigned sleep_ns = 0,
                                          long long limit_cycles = WAIT_LIMIT_CYCLES) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned ns = 32;
  for (;;) {
    if (sleep_ns) __nanosleep(ns);
    if (mbar_try_wait(bar, parity)) return true;
    if (ns < sleep_ns) ns *= 2;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit_cycles) break;
  }
  *abort_flag = 1;
  atomicCAS(&g_status, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               int code, long long limit_cycles = WAIT_LIMIT_CYCLES) {
  return mbar_wait(bar, parity, abort_flag, code, 0, limit_cycles);
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Makes generic-proxy shared-memory writes of this thread visible to the async proxy (tcgen05.mma
// operand reads, bulk copies).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- TMEM ----------------------------------------------------------------------------------
// Executed by one full warp.  ncols: power of two in [32, 512].  The base address is written to
// *result_smem.
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// ---- descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address >> 4 in bits [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48), layout type
// in [61,64) with 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of tcgen05.mma kind::f16 with bf16 operands and fp32 accumulation:
// c_format F32 (1) at bit 4, a/b format BF16 (1) at bits 7 / 10, a/b major (0 = K-major,
// 1 = MN-major) at bits 15 / 16, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the descriptors given as 32-bit halves.  Start address and leading byte offset sit in
// the low word, so an issuing thread that walks through shared memory only adds to one 32-bit
// register per operand; the high word (stride byte offset, version, swizzle mode) is a constant.
// Matters because ONE thread issues every MMA of a block: each instruction it spends between two
// tcgen05.mma shows up directly in the MMA rate (an M128 N64 K16 MMA takes 48 cycles).
__host__ __device__ constexpr uint32_t desc_sw128_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint32_t desc_sw128_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3FFFF) >> 4) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
}
__device__ __forceinline__ void mma_bf16_ss_lo(uint32_t tmem_d, uint32_t alo, uint32_t ahi, uint32_t blo,
                                               uint32_t bhi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      :
      : "r"(tmem_d), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 32 lanes x 32 columns of fp32 accumulators: thread i of the warp receives columns
// [col, col + 32) of TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- small helpers -------------------------------------------------------------------------------
// Bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned); the
// copy engine adds `bytes` to the transaction count of the mbarrier when the data has landed.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 ldg16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
// Streaming 16-byte load that stays out of L1 (ld.global.cg): for data that is read once and would
// only evict the source rows the producers keep re-reading from the small L1.
__device__ __forceinline__ uint4 ldcg16(const void* p) {
  return __ldcg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void sts16(uint32_t saddr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void bf16x2_fma(uint32_t packed, float w, float& a0, float& a1) {
  a0 = fmaf(w, __uint_as_float(packed << 16), a0);
  a1 = fmaf(w, __uint_as_float(packed & 0xFFFF0000u), a1);
}
// acc.{x,y} += w.{x,y} * (the two bf16 of `packed` widened to fp32), one packed-fp32 FMA.
__device__ __forceinline__ void ffma2_bf16x2(float2& acc, const float2& w, uint32_t packed) {
  const float2 v = make_float2(__uint_as_float(packed << 16), __uint_as_float(packed & 0xFFFF0000u));
  asm("fma.rn.f32x2 %0, %1, %2, %0;"
      : "+l"(reinterpret_cast<unsigned long long&>(acc))
      : "l"(reinterpret_cast<const unsigned long long&>(w)),
        "l"(reinterpret_cast<const unsigned long long&>(v)));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace tc
}  // namespace mc
