// Inline-PTX wrappers for sm_100a: mbarrier, TMA tiled copies, tcgen05 (alloc, mma,
// commit, ld/st), proxy fences, and the UMMA descriptor encodings.  Every wait is
// bounded: when its limit runs out it records a code in the caller's status word,
// raises the CTA-wide abort flag and returns, so a broken pipeline ends instead of
// hanging the GPU.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace evo {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// The same test with a suspend-time hint: the hardware parks the thread until the phase completes
// or the hint (nanoseconds, capped by the system) runs out, so a waiting warp does not compete
// for issue slots with the warps that do the arithmetic.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(1000000u)
      : "memory");
  return ok != 0;
}

// About one second at B200 clocks.
constexpr long long kWaitLimitCycles = 2000000000LL;

// Bounded wait.  `abort_flag` lives in shared memory and is shared by the CTA: once any
// wait has failed, all later waits fall through at once.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_parked(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}

// The same primitives on 32-bit shared-window addresses (smem_u32 of the barrier, computed once):
// no generic-pointer arithmetic or address-space conversion per call, and a wait loop that looks
// at the clock and the abort flag only after every 1024 unsuccessful tries.
__device__ __forceinline__ void mbar_arrive_s(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_s(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_s(uint32_t bar, uint32_t parity) {
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
// Up to 1024 suspended tries in one tight loop (a waiting warp shares its scheduler with warps that
// have arithmetic to issue: every instruction of the polling loop takes an issue slot from them).
__device__ __forceinline__ bool mbar_try_wait_burst_s(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .u32 c;\n\t"
      "mov.u32 c, 0;\n"
      "EVO_W_AGAIN:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "@p bra EVO_W_DONE;\n\t"
      "add.u32 c, c, 1;\n\t"
      "setp.lt.u32 p, c, 1024;\n\t"
      "@p bra EVO_W_AGAIN;\n\t"
      "setp.ne.u32 p, 0, 0;\n"
      "EVO_W_DONE:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(1000000u)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_slow_s(uint32_t bar, uint32_t parity, uint32_t abort_flag_s, int* status, int code) {
  long long t0 = 0;
  for (uint32_t round = 0;; ++round) {
    if (mbar_try_wait_burst_s(bar, parity)) return true;
    uint32_t ab;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(ab) : "r"(abort_flag_s));
    if (ab) return false;
    if (round == 0) {
      t0 = clock64();
    } else if (clock64() - t0 > kWaitLimitCycles) {
      asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_flag_s), "r"(1u) : "memory");
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait_s(uint32_t bar, uint32_t parity, uint32_t abort_flag_s, int* status, int code) {
  if (mbar_try_wait_s(bar, parity)) return true;
  return mbar_wait_slow_s(bar, parity, abort_flag_s, status, code);
}

// Generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_async_shared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- TMA (tiled, no multicast)
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until the bulk groups of this thread have finished READING their shared-memory source.
__device__ __forceinline__ void tma_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Wait until the bulk groups of this thread have completed entirely.
__device__ __forceinline__ void tma_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------- tcgen05: TMEM management
// Whole-warp instructions (.sync.aligned): call with all 32 lanes converged.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------- tcgen05: MMA
// D[tmem] (+)= A[smem] * B[smem];  issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every tcgen05 op this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Instruction descriptor for kind::f16 (bf16 or fp16 operands, fp32 accumulate).
//   [4,6) D format: 1 = f32      [7,10) A format: 0 = f16, 1 = bf16     [10,13) B format
//   [15] A major: 0 = K, 1 = MN  [16] B major                            [17,23) N>>3   [24,29) M>>4
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, bool a_mn_major, bool b_mn_major, int M, int N) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// Shared-memory matrix descriptor.
//   [0,14) start address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version = 1 (Blackwell)   [61,64) swizzle: 0 none, 2 = 128B, 4 = 64B, 6 = 32B
// Swizzled K-major tiles: rows of `swizzle` bytes, 8-row atoms, SBO = 8 * swizzle (next 8 rows).
// Swizzled MN-major tiles: SBO = next 8 K-rows, LBO = next `swizzle`-byte block along M/N.
constexpr uint32_t SWZ_128B = 2, SWZ_64B = 4, SWZ_32B = 6;
// The same encoding without the start address, usable in constant expressions, and the
// assembly of a descriptor from a precomputed low word ((address >> 4) | leading-offset field)
// and high word.
__host__ __device__ constexpr uint64_t make_sdesc_const(uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swz) {
  return (static_cast<uint64_t>(lbo_bytes >> 4) << 16) | (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) |
         (static_cast<uint64_t>(swz) << 61);
}
__device__ __forceinline__ uint64_t pack_desc(uint32_t lo, uint32_t hi) {
  return static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
}
__host__ __device__ constexpr uint32_t swizzle_code_for_row_bytes(int row_bytes) {
  return row_bytes == 128 ? SWZ_128B : (row_bytes == 64 ? SWZ_64B : SWZ_32B);
}

// ---------------------------------------------------------------- tcgen05: TMEM <-> registers
// 32x32b shape: lane l of the warp reads TMEM lane (base_lane + l), N consecutive 32-bit columns.
// A warp may only touch the 32 TMEM lanes of its own quarter: lanes 32*(warp_id % 4) ...
#define EVO_R4(r, i) "=r"(r[i]), "=r"(r[i + 1]), "=r"(r[i + 2]), "=r"(r[i + 3])
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : EVO_R4(r, 0), EVO_R4(r, 4), EVO_R4(r, 8), EVO_R4(r, 12), EVO_R4(r, 16), EVO_R4(r, 20), EVO_R4(r, 24),
        EVO_R4(r, 28)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : EVO_R4(r, 0), EVO_R4(r, 4), EVO_R4(r, 8), EVO_R4(r, 12)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : EVO_R4(r, 0), EVO_R4(r, 4)
               : "r"(taddr)
               : "memory");
}
#undef EVO_R4
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[N]) {
  static_assert(N == 8 || N == 16 || N == 32, "unsupported TMEM load width");
  if constexpr (N == 32) tmem_ld32(taddr, r);
  else if constexpr (N == 16) tmem_ld16(taddr, r);
  else tmem_ld8(taddr, r);
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

#define EVO_I4(r, i) "r"(r[i]), "r"(r[i + 1]), "r"(r[i + 2]), "r"(r[i + 3])
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::EVO_I4(r, 0), EVO_I4(r, 4), EVO_I4(r, 8), EVO_I4(r, 12), EVO_I4(r, 16), EVO_I4(r, 20), EVO_I4(r, 24),
      EVO_I4(r, 28), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
               ::EVO_I4(r, 0), EVO_I4(r, 4), "r"(taddr)
               : "memory");
}
#undef EVO_I4

// ---------------------------------------------------------------- predicated global loads
// A load whose value is needed much later must not be followed by a select on its result: the
// select would wait for the load where it stands.  These write the destination only when `pred`
// holds and leave `dflt` in it otherwise; the address is not touched when `pred` is false.
__device__ __forceinline__ uint32_t ldg_u32_if(const void* p, bool pred) {
  uint32_t v = 0u;
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t@q ld.global.u32 %0, [%1];\n\t}"
               : "+r"(v) : "l"(p), "r"((int)pred));
  return v;
}
__device__ __forceinline__ uint32_t ldg_u16_if(const void* p, bool pred) {
  uint32_t v = 0u;
  asm volatile("{\n\t.reg .pred q;\n\t.reg .b16 h;\n\tsetp.ne.b32 q, %2, 0;\n\tmov.b16 h, 0;\n\t"
               "@q ld.global.u16 h, [%1];\n\t@q cvt.u32.u16 %0, h;\n\t}"
               : "+r"(v) : "l"(p), "r"((int)pred));
  return v;
}
__device__ __forceinline__ uint32_t ldg_u8_if(const void* p, bool pred) {
  uint32_t v = 0u;
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t@q ld.global.u8 %0, [%1];\n\t}"
               : "+r"(v) : "l"(p), "r"((int)pred));
  return v;
}

// ---------------------------------------------------------------- shared-memory access by 32-bit address
// A load through a generic pointer that happens to point into shared memory is a generic load: it
// pays the address-space check and 64-bit address arithmetic, and the hardware tracks it like a
// global load.  These take the 32-bit shared-window address (smem_u32) and stay LDS / STS.
__device__ __forceinline__ float lds_f32(uint32_t saddr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
  return v;
}
__device__ __forceinline__ uint16_t lds_u16(uint32_t saddr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(saddr));
  return v;
}
__device__ __forceinline__ float4 lds_v4f(uint32_t saddr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t saddr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(saddr), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_v4(uint32_t saddr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// ---------------------------------------------------------------- small math / sync helpers
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed fp32x2 arithmetic (sm_100): one instruction works on two floats held in a 64-bit
// register pair; halves the issue slots of the element-wise softmax math.
struct F2 {
  unsigned long long v;
};
__device__ __forceinline__ F2 f2_make(float lo, float hi) {
  F2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ F2 f2_from_bits(uint32_t lo, uint32_t hi) {
  F2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_get(F2 a, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.v));
}
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
  F2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
  return r;
}
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) {
  F2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Move registers between the warps of a CTA (whole-warp instructions).  The requests of all
// warps must sum to at most the launch-time pool, or `inc` blocks for ever.
template <int N> __device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// Named barrier among `nthreads` threads (ids 1..15; id 0 is __syncthreads).
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------- leader-predicated commit
// For a warp that runs with all 32 lanes converged and predicates only the instruction that must be
// issued by a single thread (`leader` is non-zero in exactly one lane).
__device__ __forceinline__ void mma_commit_if_s(uint32_t leader, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar), "r"(leader)
      : "memory");
}
// ---------------------------------------------------------------- TMA on 32-bit shared-window addresses
__device__ __forceinline__ void tma_load_5d_s(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                              int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_s(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                              int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_s(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Tiled reduction shared -> global: global[tile] += shared[tile] (type and tile from the map).
__device__ __forceinline__ void tma_reduce_add_4d_s(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d_s(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---------------------------------------------------------------- MMA groups in one statement
// The compiler spends dozens of instructions on every separately written tcgen05.mma (descriptor
// assembly, moves into uniform registers).  A warp that issues many small MMAs next to busy
// arithmetic warps is bound by that, so the fixed groups of the backward are written out: operands
// in, a handful of adds, the MMAs.  All are issued by the calling thread (call from one lane).
// Four D[tmem] (+)= A[tmem] * B[smem] with A advancing 16 columns and B advancing `b_step` descriptor
// units per MMA; the first overwrites D unless `acc_first`.
__device__ __forceinline__ void mma_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t b_step,
                                          uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 d0, d1, d2, d3;\n\t.reg .b32 a1, a2, a3, l1, l2, l3;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 l1, %2, %4;\n\tadd.u32 l2, l1, %4;\n\tadd.u32 l3, l2, %4;\n\t"
      "add.u32 a1, %1, 16;\n\tadd.u32 a2, %1, 32;\n\tadd.u32 a3, %1, 48;\n\t"
      "mov.b64 d0, {%2, %3};\n\tmov.b64 d1, {l1, %3};\n\tmov.b64 d2, {l2, %3};\n\tmov.b64 d3, {l3, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d0, %5, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], d1, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], d2, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], d3, %5, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(b_step), "r"(idesc), "r"(acc_first)
      : "memory");
}
// The same with two MMAs (A advancing 16 columns, B advancing `b_step` units).
__device__ __forceinline__ void mma_ts_x2(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t b_step,
                                          uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 d0, d1;\n\t.reg .b32 a1, l1;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 l1, %2, %4;\n\t"
      "add.u32 a1, %1, 16;\n\t"
      "mov.b64 d0, {%2, %3};\n\tmov.b64 d1, {l1, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d0, %5, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], d1, %5, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(b_step), "r"(idesc), "r"(acc_first)
      : "memory");
}
// Two D[tmem] = A[smem] * B[smem] over two K slices (descriptors advance by `k_step` units), then a
// commit to `bar` (and to `bar2` if non-zero).
__device__ __forceinline__ void mma_ss_x2_commit(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t k_step,
                                                 uint32_t idesc, uint32_t bar, uint32_t bar2) {
  asm volatile(
      "{\n\t.reg .pred f, t, c;\n\t.reg .b64 a0, a1, b0, b1;\n\t.reg .b32 x, y;\n\t"
      "setp.ne.b32 f, 0, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "setp.ne.b32 c, %7, 0;\n\t"
      "add.u32 x, %1, %4;\n\tadd.u32 y, %2, %4;\n\t"
      "mov.b64 a0, {%1, %3};\n\tmov.b64 a1, {x, %3};\n\tmov.b64 b0, {%2, %3};\n\tmov.b64 b1, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a0, b0, %5, f;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %5, t;\n\t"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
      "@c tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(k_step), "r"(idesc), "r"(bar), "r"(bar2)
      : "memory");
}
// The same over four K slices.
__device__ __forceinline__ void mma_ss_x4_commit(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t k_step,
                                                 uint32_t idesc, uint32_t bar, uint32_t bar2) {
  asm volatile(
      "{\n\t.reg .pred f, t, c;\n\t.reg .b64 da, db;\n\t.reg .b32 x, y;\n\t"
      "setp.ne.b32 f, 0, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "setp.ne.b32 c, %7, 0;\n\t"
      "mov.u32 x, %1;\n\tmov.u32 y, %2;\n\t"
      "mov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, f;\n\t"
      "add.u32 x, x, %4;\n\tadd.u32 y, y, %4;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, t;\n\t"
      "add.u32 x, x, %4;\n\tadd.u32 y, y, %4;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, t;\n\t"
      "add.u32 x, x, %4;\n\tadd.u32 y, y, %4;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, t;\n\t"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
      "@c tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(k_step), "r"(idesc), "r"(bar), "r"(bar2)
      : "memory");
}
// Eight D[tmem] = A[smem] * B[smem] (the first overwrites), A and B descriptors advancing by
// `a_step` / `b_step` units per MMA, different high words.
__device__ __forceinline__ void mma_ss_x8(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t a_step, uint32_t b_lo,
                                          uint32_t b_hi, uint32_t b_step, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t.reg .b32 x, y;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "mov.u32 x, %1;\n\tmov.u32 y, %4;\n\t"
      "mov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "add.u32 x, x, %3;\n\tadd.u32 y, y, %6;\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
      "add.u32 x, x, %3;\n\tadd.u32 y, y, %6;\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
      "add.u32 x, x, %3;\n\tadd.u32 y, y, %6;\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
      "add.u32 x, x, %3;\n\tadd.u32 y, y, %6;\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
      "add.u32 x, x, %3;\n\tadd.u32 y, y, %6;\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
      "add.u32 x, x, %3;\n\tadd.u32 y, y, %6;\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t"
      "add.u32 x, x, %3;\n\tadd.u32 y, y, %6;\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %7, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(a_step), "r"(b_lo), "r"(b_hi), "r"(b_step), "r"(idesc)
      : "memory");
}

// Non-blocking arrival on a named barrier that other threads wait on with named_bar_sync.
__device__ __forceinline__ void named_bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace ptx
}  // namespace evo
