// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM wrappers,
// bounded waits with a status word, vector load/store helpers.
//
// Every wait in this library is bounded.  When a wait gives up it records where in a
// status word that the host reads after the stream has drained; the kernel then runs to
// its normal end (frees TMEM, drains its bulk copies) so that the context stays usable.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define AX_API extern "C" __attribute__((visibility("default")))

namespace ax {

// ---------------------------------------------------------------- status word
// status[0] = first error code (0 = ok), status[1] = detail (where), status[2] = block id,
// status[3] = wait budget in microseconds set by the host (0 = the built-in budgets)
enum StatusCode : int {
  kOk = 0,
  kWaitTimeout = 1,   // an mbarrier / flag wait ran out
  kBadArgument = 2,
  kPeerTimeout = 3,   // a wait on another rank's signal ran out
};

__device__ __forceinline__ void set_status(int* status, int code, int detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0, code) == 0) {
      status[1] = detail;
      status[2] = (int)blockIdx.x;
    }
  }
}

// ---------------------------------------------------------------- bounds-checked debug build
// Compiled with -DAX_BOUNDS=1 (relocatable device code, its own shared object) the kernels check the
// indices they compute before they use them: AX_INB(i, width, n, where) is true when elements
// [i, i + width) lie inside an n-element extent; otherwise it records {code 4, where, index,
// extent} once in a word that the host reads with ax_bounds_read and returns false, and the caller
// skips the access, so a wrong index is reported instead of reading or writing memory it should
// not.  In the normal build the macro is the constant `true` and the checks vanish.
#ifdef AX_BOUNDS
extern __device__ int g_bounds_word[6];   // code, where, index lo/hi 32 bits, extent lo/hi 32 bits
__device__ __forceinline__ bool in_bounds(long i, long width, long n, int where) {
  if (i >= 0 && i + width <= n) return true;
  if (atomicCAS(&g_bounds_word[0], 0, 4) == 0) {
    g_bounds_word[1] = where;
    g_bounds_word[2] = (int)(i & 0xffffffffL); g_bounds_word[3] = (int)(i >> 32);
    g_bounds_word[4] = (int)(n & 0xffffffffL); g_bounds_word[5] = (int)(n >> 32);
  }
  return false;
}
#define AX_INB(i, width, n, where) ax::in_bounds((long)(i), (long)(width), (long)(n), (where))
#else
#define AX_INB(i, width, n, where) true
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait budget for on-chip waits (TMA landing, MMA retiring): far above any legal latency.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s

// The budget a wait works with: the host's value from the status word when it set one (tests make
// a wait run out in milliseconds that way), else `builtin_ns`.  Read on the slow path only.
__device__ __forceinline__ uint64_t wait_budget_ns(const int* status, uint64_t builtin_ns) {
  if (status != nullptr) {
    const int us = *(const volatile int*)(status + 3);
    if (us > 0) return (uint64_t)us * 1000ull;
  }
  return builtin_ns;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint32_t lane_id() {
  return threadIdx.x & 31;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// mbarrier.try_wait may carry a hint of how long (ns) the hardware may keep the waiting thread
// suspended before it returns; the thread wakes when the phase completes.  0 compiles the plain
// form, which returns after the hardware's own short limit so that the loop around it polls more
// often.  Measured both ways on one B200: the flash kernels gain 2 % from the plain form, the
// 8192^3 GEMM loses 4 % (the polling takes issue slots from the warps that work).
#ifndef AX_SUSPEND_HINT_NS
#define AX_SUSPEND_HINT_NS 20000
#endif
constexpr uint32_t kSuspendHintNs = AX_SUSPEND_HINT_NS;

// Bounded wait.  `dead` is a shared-memory flag of the CTA: once any wait of the CTA has
// given up, all later waits return at once so that the CTA drains quickly.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* dead,
                                          int* status, int where) {
  uint32_t ok = 0;
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    if (kSuspendHintNs != 0) {
      asm volatile(
          "{\n\t"
          ".reg .pred P;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
          "selp.b32 %0, 1, 0, P;\n\t"
          "}\n"
          : "=r"(ok)
          : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
          : "memory");
    } else {
      asm volatile(
          "{\n\t"
          ".reg .pred P;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
          "selp.b32 %0, 1, 0, P;\n\t"
          "}\n"
          : "=r"(ok)
          : "r"(smem_u32(bar)), "r"(parity)
          : "memory");
    }
    if (ok) return true;
    if (++spins >= 16) {
      if (*dead) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > wait_budget_ns(status, kWaitBudgetNs)) {
        *dead = 1;
        set_status(status, kWaitTimeout, where);
        return false;
      }
      spins = 0;
    }
  }
}

// ---------------------------------------------------------------- TMA (plain per-CTA loads and stores)
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
        "r"(w)
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x,
                                             int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"((uint64_t)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x,
                                             int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               :
               : "l"((uint64_t)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
template <int kCols>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "n"(kCols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int kCols>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kCols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (count 1) on an mbarrier of this CTA once all tcgen05 ops issued so far have retired.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2i and 2i+1) run one MMA together: each holds half of the rows of
// A and of the accumulator and half of the columns of B; the even ("leader") CTA issues the
// instruction, the hardware reads the same shared-memory offsets in both CTAs.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) as seen in CTA `rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive (count 1) on an mbarrier given by its shared::cluster address (this or the peer CTA).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// Plain (no multicast) tiled load into THIS CTA's shared memory whose completion bytes are
// counted on an mbarrier of either CTA of the pair (given by its shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
template <int kCols>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "n"(kCols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int kCols>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kCols)
               : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the pair: M = 256 (128 rows per CTA), B split by columns.
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (count 1) on the mbarrier at the same shared-memory offset in BOTH CTAs of the pair once
// all tcgen05 ops issued so far by this thread have retired.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp reads lane (base+i), columns c..c+31.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle, 16-bit elements.
//  K-major : tile stored as rows of 64 elements (128 B), 8-row groups 1024 B apart.
//  MN-major: tile stored as K-rows of 64 MN-elements (128 B); 8 K-rows = 1024 B (SBO);
//            consecutive 64-element MN slabs are `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation.
//  fmt: 0 = fp16, 1 = bf16; major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int fmt, int m, int n, int a_major,
                                                      int b_major) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_major << 15) |
         ((uint32_t)b_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------- small numeric helpers
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float t = tanhf(u);
  float du = k0 * (1.f + 3.f * k1 * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }

enum Act : int { kActNone = 0, kActRelu = 1, kActGelu = 2, kActSigmoid = 3, kActTanh = 4, kActSilu = 5 };

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case kActRelu: return x > 0.f ? x : 0.f;
    case kActGelu: return gelu_tanh(x);
    case kActSigmoid: return sigmoidf_(x);
    case kActTanh: return tanhf(x);
    case kActSilu: return siluf_(x);
    default: return x;
  }
}

// Activation over a 64-value accumulator chunk with ONE branch on `act`: a switch per element
// costs a chain of taken branches each, which an epilogue warp (alone on its scheduler) cannot
// hide -- measured at 4 us per chunk against 0.5 us for the rest of the chunk's work.
__device__ __forceinline__ void apply_act_chunk(uint32_t (&r)[64], int act) {
  switch (act) {
    case kActRelu:
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] = __float_as_uint(fmaxf(__uint_as_float(r[j]), 0.f));
      break;
    case kActGelu:
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] = __float_as_uint(gelu_tanh(__uint_as_float(r[j])));
      break;
    case kActSigmoid:
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] = __float_as_uint(sigmoidf_(__uint_as_float(r[j])));
      break;
    case kActTanh:
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] = __float_as_uint(tanhf(__uint_as_float(r[j])));
      break;
    case kActSilu:
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] = __float_as_uint(siluf_(__uint_as_float(r[j])));
      break;
    default: break;
  }
}

// Bias (fp32 or bf16, kind 1 / 2) added to a 64-column chunk starting at column n0 of N columns;
// the kind and the range test are hoisted out of the element loop.
__device__ __forceinline__ void add_bias_chunk(uint32_t (&r)[64], const void* bias, int kind, int n0, int N) {
  if (kind == 0) return;
  if (n0 + 64 <= N) {
    if (kind == 1) {
      const float4* b4 = reinterpret_cast<const float4*>((const float*)bias + n0);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float4 b = __ldg(b4 + j);
        r[4 * j + 0] = __float_as_uint(__uint_as_float(r[4 * j + 0]) + b.x);
        r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + b.y);
        r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + b.z);
        r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + b.w);
      }
    } else {
      const uint4* b8 = reinterpret_cast<const uint4*>((const __nv_bfloat16*)bias + n0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 b = __ldg(b8 + j);
        const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[k]);
          const float2 f = __bfloat1622float2(h);
          r[8 * j + 2 * k + 0] = __float_as_uint(__uint_as_float(r[8 * j + 2 * k + 0]) + f.x);
          r[8 * j + 2 * k + 1] = __float_as_uint(__uint_as_float(r[8 * j + 2 * k + 1]) + f.y);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 64; ++j) {
    const int n = n0 + j;
    float b = 0.f;
    if (n < N) b = kind == 1 ? __ldg((const float*)bias + n) : __bfloat162float(((const __nv_bfloat16*)bias)[n]);
    r[j] = __float_as_uint(__uint_as_float(r[j]) + b);
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace ax

// ---------------------------------------------------------------- host helpers
namespace axh {
// Encodes a tiled tensor map through the driver entry point (resolved at run time so that
// the library links without libcuda).  Returns 0 on success.
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);
int sm_count();
}  // namespace axh
