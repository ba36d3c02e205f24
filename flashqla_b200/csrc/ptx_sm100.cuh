// Thin inline-PTX wrappers for the Blackwell (sm_100a) primitives the kernels use:
// mbarriers with BOUNDED waits, TMA tiled copies (cp.async.bulk.tensor), tensor memory
// (tcgen05.alloc / ld / st) and the 5th-generation tensor-core MMA (tcgen05.mma) with its shared
// memory / instruction descriptors.  Every copy has one destination CTA (no clusters are launched).
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "common.cuh"

namespace qla {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.b32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after `kSpinLimit` polls or `kWaitLimitNs` of wall time, whichever comes
// first (each try_wait itself blocks for a hardware-defined interval, so the poll count alone does not
// bound the time), records the failure in *status and returns false so that the caller can leave its
// loop.  A healthy kernel never gets near the limit.  The recorded word is
//   code | parity << 16 | warp << 20      (callers put the barrier's index into bits 8..15 of `code`).
// The first poll is inlined (the barrier has usually completed already); the polling loop is a single
// non-inlined copy: there are dozens of call sites and the per-chunk code of the chunk kernels has to
// fit the instruction cache.
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void record_wait_failure(int* status, int code, uint32_t parity) {
  if (status != nullptr) atomicCAS(status, 0, code | static_cast<int>(parity << 16) | static_cast<int>((threadIdx.x >> 5) << 20));
}
// The polling loop itself; `limit_ns` is kWaitLimitNs everywhere except in the self-test of this very path.
__device__ __forceinline__ bool mbar_wait_polling(uint64_t* bar, uint32_t parity, int* status, int code,
                                                  unsigned long long limit_ns) {
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0)
        return false;  // another role already failed: do not keep the SM busy
      if (global_timer_ns() - t0 > limit_ns) break;
    }
  }
  record_wait_failure(status, code, parity);
  return false;
}
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int* status, int code) {
  return mbar_wait_polling(bar, parity, status, code, kWaitLimitNs);
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, status, code);
}

// Low-latency variant for a single latency-critical thread (the MMA issuer): polls with
// mbarrier.test_wait, which never suspends the thread, so the wake-up is not delayed by the
// hardware's try_wait back-off.  Still bounded.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
static __device__ __noinline__ bool mbar_spin_slow(uint64_t* bar, uint32_t parity, int* status, int code) {
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t i = 0; i < (kSpinLimit << 4); ++i) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((i & 4095u) == 4095u) {
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) break;
    }
  }
  record_wait_failure(status, code, parity);
  return false;
}
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_test_wait(bar, parity)) return true;
  return mbar_spin_slow(bar, parity, status, code);
}

// Same wait executed by a converged warp; the verdict is made warp-uniform so that no lane leaves a
// loop alone (later __syncwarp / .sync.aligned instructions need the whole warp).
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* status, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, status, code)) != 0;
}

// Wait executed by a CONVERGED warp, verdict warp-uniform.  The first poll is inline and not voted on:
// the lanes of a converged warp execute the try_wait as one instruction on one barrier word and see the
// same answer, so either all of them return here or all of them enter the (non-inlined) polling loop,
// whose vote makes the verdict uniform even at the edge of the time limit.
static __device__ __noinline__ bool mbar_wait_warp_slow(uint64_t* bar, uint32_t parity, int* status, int code) {
  return __all_sync(__activemask(), mbar_wait_slow(bar, parity, status, code)) != 0;
}
__device__ __forceinline__ bool mbar_wait_warp_call(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_warp_slow(bar, parity, status, code);
}

__device__ __forceinline__ float ex2(float x) {  // 2^x, approximate (the MUFU behind __expf)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------------------ fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------------------ TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// Tiled 3-D load: coordinates are (x = innermost element, y, z); x * elem_size must be a multiple
// of 16 bytes.  Completion is signalled on `bar` with the byte count of the box.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Bring a box into L2 only (no shared-memory destination, no completion tracking).
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* m, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* src, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until the bulk stores of all committed groups have finished READING shared memory.
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------------------ tensor memory
// Allocate `ncols` (power of two >= 32) TMEM columns; executed by ONE full warp.  The base address
// is written to *dst_smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 lanes x 32 bit: thread i of the warp reads lane (base lane + i); register j = column + j.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 256 bit fragments: the warp reads lanes L .. L + 15 (L = lane field of the address: the first or
// the second half of the warp's 32-lane partition, i.e. the rows of an M = 64 accumulator placed at lane offset
// 0 or 16) and thread t = 4 g + c receives, per group j of eight columns, the four values
//   r[4j + 0..1] = (lane L + g,     columns 8j + 2c, 8j + 2c + 1)
//   r[4j + 2..3] = (lane L + g + 8, the same columns)
// - the accumulator layout of mma.sync m16n8 tiles.
__device__ __forceinline__ void tmem_ld_frag8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_frag4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_frag2(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets
// (all >> 4), descriptor version 1 at bit 46, swizzle mode at bits 61-63 (2 = 128-byte swizzle).
// For 128B-swizzled tiles the tile base must be 1024-byte aligned; stepping the start address by
// 32 bytes moves 16 bf16 along the contiguous direction inside the swizzle atom.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

enum : uint32_t { kMajorK = 0, kMajorMN = 1 };
enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1 };

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation.
__host__ __device__ constexpr uint32_t mma_idesc(uint32_t m, uint32_t n, uint32_t fmt, uint32_t a_major,
                                                  uint32_t b_major) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_major << 15) | (b_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is M x 16 (K-major, two 16-bit values per 32-bit column).
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// Make `bar` complete one arrival once every MMA issued so far by this thread has finished
// (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// ---- whole products issued by a CONVERGED warp.
// A tcgen05.mma is issued by one thread, but when that thread sits in a divergent branch every operand
// lives in per-thread registers and has to be moved to uniform registers one by one: measured ~55-68
// cycles of issue per instruction, more than the tensor pipe needs for N <= 128.  Issued from a
// converged warp with the leader picked by elect.sync INSIDE the asm block, the operand arithmetic stays
// on the uniform datapath and the cost drops to the pipe's own (34 cycles at N = 64, 68 at N = 128).
// Descriptor steps are 32-bit adds on the low word (the 14-bit address field never carries).
// All steps are in units of 16 bytes.  `JUMP` replaces `STEP` between k-steps 3 and 4 (the second
// 64-element half of a 128-wide operand).  Every block ends with up to two tcgen05.commit on the
// barriers whose shared-memory addresses are passed in (0 = none), so that a product and its completion
// signal cost one leader election.
#define QLA_UMMA_COMMITS(B1, B2)                                                                      \
  "setp.ne.b32 c1, " B1 ", 0;\nsetp.ne.b32 c2, " B2 ", 0;\nand.pred c1, c1, e;\nand.pred c2, c2, e;\n"   \
  "@c1 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [" B1 "];\n"              \
  "@c2 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [" B2 "];\n"
#define QLA_UMMA_SS_STEP(SA, SB)                                                                     \
  "add.u32 alo, alo, " SA "; add.u32 blo, blo, " SB "; mov.b64 da, {alo, ahi}; mov.b64 db, {blo, bhi};\n" \
  "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, t;\n"
#define QLA_UMMA_SS_HEAD                                                                              \
  "{\n.reg .pred p, t, e, c1, c2;\n.reg .b32 alo, ahi, blo, bhi;\n.reg .b64 da, db;\n"                         \
  "elect.sync _|e, 0xffffffff;\nsetp.ne.b32 p, %4, 0;\nsetp.eq.b32 t, 0, 0;\n"                         \
  "mov.b64 {alo, ahi}, %1;\nmov.b64 {blo, bhi}, %2;\n"                                                 \
  "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
// D[tmem] (+)= A[smem] B[smem], K = 64 (four instructions).
template <int A_STEP, int B_STEP>
__device__ __forceinline__ void umma_ss_k64(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            bool accumulate, uint32_t commit1 = 0, uint32_t commit2 = 0) {
  asm volatile(QLA_UMMA_SS_HEAD QLA_UMMA_SS_STEP("%5", "%6") QLA_UMMA_SS_STEP("%5", "%6") QLA_UMMA_SS_STEP("%5", "%6")
               QLA_UMMA_COMMITS("%7", "%8") "}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate)),
                 "n"(A_STEP), "n"(B_STEP), "r"(commit1), "r"(commit2)
               : "memory");
}
// D[tmem] (+)= A[smem] B[smem], K = 128 (eight instructions).
template <int A_STEP, int A_JUMP, int B_STEP, int B_JUMP>
__device__ __forceinline__ void umma_ss_k128(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             bool accumulate, uint32_t commit1 = 0, uint32_t commit2 = 0) {
  asm volatile(QLA_UMMA_SS_HEAD QLA_UMMA_SS_STEP("%5", "%6") QLA_UMMA_SS_STEP("%5", "%6") QLA_UMMA_SS_STEP("%5", "%6")
               QLA_UMMA_SS_STEP("%7", "%8") QLA_UMMA_SS_STEP("%5", "%6") QLA_UMMA_SS_STEP("%5", "%6") QLA_UMMA_SS_STEP("%5", "%6")
               QLA_UMMA_COMMITS("%9", "%10") "}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate)),
                 "n"(A_STEP), "n"(B_STEP), "n"(A_JUMP), "n"(B_JUMP), "r"(commit1), "r"(commit2)
               : "memory");
}
#undef QLA_UMMA_SS_STEP
#undef QLA_UMMA_SS_HEAD
#define QLA_UMMA_TS_STEP(SB)                                                                         \
  "add.u32 aa, aa, 8; add.u32 blo, blo, " SB "; mov.b64 db, {blo, bhi};\n"                             \
  "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], db, %3, t;\n"
#define QLA_UMMA_TS_HEAD                                                                              \
  "{\n.reg .pred p, t, e, c1, c2;\n.reg .b32 aa, blo, bhi;\n.reg .b64 db;\n"                                   \
  "elect.sync _|e, 0xffffffff;\nsetp.ne.b32 p, %4, 0;\nsetp.eq.b32 t, 0, 0;\n"                         \
  "mov.b32 aa, %1;\nmov.b64 {blo, bhi}, %2;\n"                                                         \
  "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
// D[tmem] (+)= A[tmem] B[smem], K = 64: A advances 8 TMEM columns (16 values of 16 bits) per instruction.
template <int B_STEP>
__device__ __forceinline__ void umma_ts_k64(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            bool accumulate, uint32_t commit1 = 0, uint32_t commit2 = 0) {
  asm volatile(QLA_UMMA_TS_HEAD QLA_UMMA_TS_STEP("%5") QLA_UMMA_TS_STEP("%5") QLA_UMMA_TS_STEP("%5")
               QLA_UMMA_COMMITS("%6", "%7") "}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate)), "n"(B_STEP),
                 "r"(commit1), "r"(commit2)
               : "memory");
}
// D[tmem] (+)= A[tmem] B[smem], K = 128.
template <int B_STEP, int B_JUMP>
__device__ __forceinline__ void umma_ts_k128(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             bool accumulate, uint32_t commit1 = 0, uint32_t commit2 = 0) {
  asm volatile(QLA_UMMA_TS_HEAD QLA_UMMA_TS_STEP("%5") QLA_UMMA_TS_STEP("%5") QLA_UMMA_TS_STEP("%5") QLA_UMMA_TS_STEP("%6")
               QLA_UMMA_TS_STEP("%5") QLA_UMMA_TS_STEP("%5") QLA_UMMA_TS_STEP("%5")
               QLA_UMMA_COMMITS("%7", "%8") "}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate)), "n"(B_STEP),
                 "n"(B_JUMP), "r"(commit1), "r"(commit2)
               : "memory");
}
#undef QLA_UMMA_TS_STEP
#undef QLA_UMMA_TS_HEAD
#undef QLA_UMMA_COMMITS
// tcgen05.commit from a converged warp (same elected lane as the umma_* helpers).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile(
      "{\n.reg .pred e;\nelect.sync _|e, 0xffffffff;\n"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(smem_u32(bar))
      : "memory");
}

// Byte offset of element (row, 16-byte chunk `c16`) inside a 128B-swizzled tile whose rows are
// 128 bytes (64 bf16) wide: chunk index is XORed with (row mod 8).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t c16) {
  return row * 128u + ((c16 ^ (row & 7u)) << 4);
}

}  // namespace ptx

// ------------------------------------------------------------------------------ host: tensor maps
// cuTensorMapEncodeTiled fetched through the runtime (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// Map over a [rows(tokens), heads, width] tensor of 16-bit elements; box = [box_rows, 1, box_width].
int make_tmap_3d(CUtensorMap* out, const void* base, uint64_t tokens, uint64_t heads, uint64_t width,
                 uint32_t box_rows, uint32_t box_width, bool swizzle128, bool is_bf16);

}  // namespace qla
