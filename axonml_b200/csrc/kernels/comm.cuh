// Device-side primitives for kernels that talk to other GPUs through peer-mapped (symmetric)
// memory over NVLink: system-scope signals with bounded waits, 16-byte peer loads/stores, and the
// NVSwitch multimem (NVLS) load-reduce / store instructions.
//
// Signal protocol: every communicator owns, on every rank, a symmetric array of 32-bit slots.
// Values only ever grow: a call with epoch e writes e (or adds 1 towards a target derived from e),
// waiters wait for "slot >= target".  Nothing is reset, so a kernel that gave up on a wait can be
// launched again.  Every wait has a time budget; on expiry the kernel records
// {code = kPeerTimeout, where, block} in the status word and carries on to its normal end.
#pragma once
#include "common.cuh"

namespace axc {
using namespace ax;

constexpr int kMaxRanks = 8;   // one NVSwitch domain (a single 8-GPU box)
constexpr uint64_t kPeerWaitBudgetNs = 1000000000ull;  // 1 s

struct Peers {
  void* buf[kMaxRanks];         // rank p's data buffer (peer-mapped)
  uint32_t* sig[kMaxRanks];     // rank p's signal array (peer-mapped)
  void* mc_buf;                 // multicast (NVLS) mapping of the data buffers, or null
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for *p >= target (wrap-safe signed compare).  Returns false on timeout.
template <bool SYS>
__device__ __forceinline__ bool wait_ge(const uint32_t* p, uint32_t target, int* status, int where) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int32_t)(v - target) >= 0) return true;
    if (++spins >= 32) {
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > wait_budget_ns(status, kPeerWaitBudgetNs)) {
        set_status(status, kPeerTimeout, where);
        return false;
      }
      spins = 0;
      __nanosleep(64);
    }
  }
}

// Cross-GPU barrier for one CTA: slot layout sig[block * world + source_rank].  Thread t < world
// signals rank t, then waits for rank t's signal.  All threads of the CTA return together.
__device__ __forceinline__ bool cta_barrier_all_ranks(const Peers& P, uint32_t epoch, int* status,
                                                      int where) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();  // also orders this CTA's earlier global writes before the signals below
  if ((int)threadIdx.x < P.world) {
    __threadfence_system();
    st_release_sys(P.sig[threadIdx.x] + blockIdx.x * P.world + P.rank, epoch);
    if (!wait_ge<true>(P.sig[P.rank] + blockIdx.x * P.world + threadIdx.x, epoch, status, where))
      ok_flag = 0;
  }
  __syncthreads();
  return ok_flag != 0;
}

// ---------------------------------------------------------------- NVLS multimem
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_ptr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b32x4(void* mc_ptr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_v4(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace axc
