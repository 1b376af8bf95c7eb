// Fused collective kernels over NVLink peer memory (NVSwitch multimem when a multicast mapping
// is available, plain peer loads/stores otherwise).
//
//  * ax_fused_allreduce : DDP bucket all-reduce (mean) fused with the GradScaler unscale and the
//    found-inf check.  Two-shot inside ONE kernel: rank r reduces slice r of every peer's bucket
//    and writes the result into slice r of every peer's bucket.
//    Replaces the per-parameter all_reduce of crates/axonml-distributed/src/ddp.rs:80-90 and the
//    separate unscale pass of crates/axonml-optim/src/grad_scaler.rs:187-206.
//  * ax_fused_rs_adamw  : FSDP gradient reduce-scatter fused with the sharded AdamW update: rank r
//    sums its shard of every peer's flat gradient, applies AdamW to its fp32 master shard and
//    moments and writes the bf16 shard.
//    Replaces fsdp.rs:259-268 (reduce-scatter whose result is dropped) + adam.rs:376-445.
//
// Synchronisation: block 0 runs the cross-GPU barriers (comm.cuh); the other blocks of the same
// GPU follow it through two local words.  The grid never exceeds the SM count, so all blocks of a
// launch are resident together.  Every wait is bounded.
#include "comm.cuh"

namespace {
using namespace ax;
using namespace axc;

constexpr int kThreads = 512;

struct Ctl {              // slots inside this rank's signal array
  uint32_t* a;            // [world] start barrier
  uint32_t* b;            // [world] end barrier (value carries a flag bit)
  uint32_t* go;           // local: start barrier passed
  uint32_t* done;         // local: blocks finished
};

__device__ __forceinline__ Ctl ctl_of(const Peers& P, int r) {
  uint32_t* s = P.sig[r];
  return Ctl{s, s + kMaxRanks, s + 2 * kMaxRanks, s + 2 * kMaxRanks + 1};
}

// Start of a collective kernel.  Returns false if a wait ran out (the caller skips its work).
// `done_base` (meaningful in thread 0 of block 0): the count of finished blocks before this launch; it
// is read before any block of this launch can have reported, and makes the end-of-launch count
// independent of how many calls this rank has made (a rank may have left a call out).
__device__ __forceinline__ bool collective_begin(const Peers& P, uint32_t epoch, int* status, uint32_t& done_base) {
  __shared__ int s_ok;
  Ctl me = ctl_of(P, P.rank);
  done_base = 0;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      s_ok = 1;
      done_base = ld_acquire_gpu(me.done);
    }
    __syncthreads();
    if ((int)threadIdx.x < P.world) {
      st_release_sys(ctl_of(P, threadIdx.x).a + P.rank, epoch);
      if (!wait_ge<true>(me.a + threadIdx.x, epoch, status, 600)) s_ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      // even on failure release the other blocks: they re-check the status word
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(me.go), "r"(epoch) : "memory");
    }
  } else {
    if (threadIdx.x == 0) s_ok = wait_ge<false>(me.go, epoch, status, 601) ? 1 : 0;
    __syncthreads();
  }
  __syncthreads();
  bool ok = s_ok != 0;
  if (status != nullptr && *(volatile int*)status != 0) ok = false;
  return ok;
}

// End of a collective kernel: all blocks report, block 0 exchanges `flag` (0/1) with every rank.
// Returns the OR of all ranks' flags (valid in block 0 only).
__device__ __forceinline__ int collective_end(const Peers& P, uint32_t epoch, int local_flag,
                                              int* status, uint32_t done_base) {
  __shared__ int s_any;
  Ctl me = ctl_of(P, P.rank);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (local_flag) atomicOr((int*)(me.done + 1), 1);        // sticky per-launch flag word
    red_release_gpu_add(me.done, 1);
  }
  if (blockIdx.x != 0) return 0;
  if (threadIdx.x == 0) {
    s_any = 0;
    wait_ge<false>(me.done, done_base + gridDim.x, status, 602);
  }
  __syncthreads();
  if ((int)threadIdx.x < P.world) {
    int mine = *(volatile int*)(me.done + 1) & 1;
    __threadfence_system();
    st_release_sys(ctl_of(P, threadIdx.x).b + P.rank, epoch * 2 + (uint32_t)mine);
    if (wait_ge<true>(me.b + threadIdx.x, epoch * 2, status, 603)) {
      uint32_t v = ld_acquire_sys(me.b + threadIdx.x);
      if (v == epoch * 2 + 1) atomicOr(&s_any, 1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *(volatile int*)(me.done + 1) = 0;
  return s_any;
}

__device__ __forceinline__ void acc_bf16x8(float (&a)[8], uint4 v) {
  float2 x = unpack_bf16x2(v.x), y = unpack_bf16x2(v.y), z = unpack_bf16x2(v.z), w = unpack_bf16x2(v.w);
  a[0] += x.x; a[1] += x.y; a[2] += y.x; a[3] += y.y; a[4] += z.x; a[5] += z.y; a[6] += w.x; a[7] += w.y;
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&a)[8]) {
  uint4 o;
  o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
  o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
  return o;
}

// Sum over ranks of the 16 bytes at byte offset `off` of every rank's buffer -> fp32 lanes.
// BF16: 8 values; F32: 4 values (lanes 4..7 unused).
template <bool BF16, bool MC>
__device__ __forceinline__ void reduce16(const Peers& P, long off, float (&a)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = 0.f;
  if (MC) {
    if (BF16) {
      acc_bf16x8(a, multimem_ld_reduce_bf16x8((const char*)P.mc_buf + off));
    } else {
      float4 v = multimem_ld_reduce_f32x4((const char*)P.mc_buf + off);
      a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
    }
  } else {
    uint4 v[kMaxRanks];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < P.world) v[p] = ld_peer_v4((const char*)P.buf[(P.rank + p) % P.world] + off);
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
      if (p < P.world) {
        if (BF16) {
          acc_bf16x8(a, v[p]);
        } else {
          a[0] += __uint_as_float(v[p].x); a[1] += __uint_as_float(v[p].y);
          a[2] += __uint_as_float(v[p].z); a[3] += __uint_as_float(v[p].w);
        }
      }
    }
  }
}

template <bool MC>
__device__ __forceinline__ void bcast16(const Peers& P, long off, uint4 v) {
  if (MC) {
    multimem_st_b32x4((char*)P.mc_buf + off, v);
  } else {
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < P.world) st_peer_v4((char*)P.buf[(P.rank + p) % P.world] + off, v);
  }
}

// bucket: n elements at byte offset base_off of every rank's buffer; n*elsize divisible by 16*world
template <bool BF16, bool MC>
__global__ void __launch_bounds__(kThreads)
fused_allreduce_kernel(const Peers P, long base_off, long n, float mul, const float* inv_scale,
                       int* found_inf, uint32_t epoch, uint32_t* epoch_dev, int* status) {
  // With a device-side call counter the launch carries no per-call argument, so it can be
  // captured in a CUDA graph and replayed: every block reads the counter at entry, block 0
  // advances it after all blocks of this launch have finished.
  if (epoch_dev != nullptr) epoch = *(volatile uint32_t*)epoch_dev + 1;
  uint32_t done_base;
  const bool ok = collective_begin(P, epoch, status, done_base);
  int bad = 0;
  if (ok) {
    const int esz = BF16 ? 2 : 4;
    const long bytes = n * esz;
    const long slice = bytes / P.world;
    const long lo = base_off + slice * P.rank;
    const float m = mul * (inv_scale ? *inv_scale : 1.f);
    for (long o = ((long)blockIdx.x * kThreads + threadIdx.x) * 16; o < slice;
         o += (long)gridDim.x * kThreads * 16) {
      float a[8];
      reduce16<BF16, MC>(P, lo + o, a);
      uint4 out;
      if (BF16) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { a[i] *= m; if (!isfinite(a[i])) bad = 1; }
        out = pack_bf16x8(a);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) { a[i] *= m; if (!isfinite(a[i])) bad = 1; }
        out = make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3]));
      }
      bcast16<MC>(P, lo + o, out);
    }
  }
  bad = __syncthreads_or(bad);
  const int any = collective_end(P, epoch, bad, status, done_base);
  if (blockIdx.x == 0 && threadIdx.x == 0 && any && found_inf) *found_inf = 1;
  if (blockIdx.x == 0 && threadIdx.x == 0 && epoch_dev != nullptr) *(volatile uint32_t*)epoch_dev = epoch;
}

// ---------------------------------------------------------------------------------------------
// One-shot sum for small vectors (tensor-parallel decode: a few KB per call, two calls per layer).
// The two-shot kernel above needs a start barrier, a reduce / broadcast round and an end barrier,
// three trips across NVLink; here every rank writes its vector into slot `rank` of every rank's
// staging area (one multimem store per 16 bytes when the switch multicasts, W peer stores
// otherwise), raises one flag per peer, waits for the W flags of its own area and adds the W
// slots it holds: one trip.  Two staging areas alternate by call parity: a rank can only reach
// call e + 2 after every peer has signalled call e + 1, i.e. after every peer has finished
// reading call e.  One CTA; the call counter lives on the device (CUDA-graph capture).
//   staging: [2 parities][W slots][slot_bytes]; flags (after the barrier words): [2][W].
constexpr int kOneShotThreads = 512;
constexpr int kOneShotFlags = 2 * kMaxRanks + 4;      // first flag word inside the signal array

template <bool BF16, bool MC>
__global__ void __launch_bounds__(kOneShotThreads)
oneshot_allreduce_kernel(const Peers P, const uint8_t* __restrict__ x, uint8_t* __restrict__ out, long bytes,
                         long slot_bytes, float mul, uint32_t* epoch_dev, int* status) {
  __shared__ int s_ok;
  const uint32_t epoch = *(volatile uint32_t*)epoch_dev + 1;
  const int par = (int)(epoch & 1u);
  const long area = (long)par * P.world * slot_bytes;
  if (threadIdx.x == 0) s_ok = 1;
  for (long o = (long)threadIdx.x * 16; o < bytes; o += (long)kOneShotThreads * 16) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + o);
    const long dst = area + (long)P.rank * slot_bytes + o;
    if (MC) {
      multimem_st_b32x4((char*)P.mc_buf + dst, v);
    } else {
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < P.world) st_peer_v4((char*)P.buf[(P.rank + p) % P.world] + dst, v);
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < P.world) {
    st_release_sys(P.sig[threadIdx.x] + kOneShotFlags + par * kMaxRanks + P.rank, epoch);
    if (!wait_ge<true>(P.sig[P.rank] + kOneShotFlags + par * kMaxRanks + threadIdx.x, epoch, status, 620)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    const uint8_t* mine = (const uint8_t*)P.buf[P.rank] + area;
    for (long o = (long)threadIdx.x * 16; o < bytes; o += (long)kOneShotThreads * 16) {
      float a[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = 0.f;
      uint4 v[kMaxRanks];
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < P.world) v[p] = ld_peer_v4(mine + (long)p * slot_bytes + o);
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p) {
        if (p < P.world) {
          if (BF16) {
            acc_bf16x8(a, v[p]);
          } else {
            a[0] += __uint_as_float(v[p].x); a[1] += __uint_as_float(v[p].y);
            a[2] += __uint_as_float(v[p].z); a[3] += __uint_as_float(v[p].w);
          }
        }
      }
      uint4 r;
      if (BF16) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] *= mul;
        r = pack_bf16x8(a);
      } else {
        r = make_uint4(__float_as_uint(a[0] * mul), __float_as_uint(a[1] * mul), __float_as_uint(a[2] * mul),
                       __float_as_uint(a[3] * mul));
      }
      *reinterpret_cast<uint4*>(out + o) = r;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *(volatile uint32_t*)epoch_dev = epoch;
}

struct AdamW {
  float lr, beta1, beta2, eps, wd, bc1, bc2, mul;
};

// grads: bf16, every rank's flat gradient at byte offset grad_off of P.buf[*]; this rank owns
// elements [rank*shard, (rank+1)*shard).
template <bool MC>
__global__ void __launch_bounds__(kThreads)
fused_rs_adamw_kernel(const Peers P, long grad_off, long shard, float* master, float* m1, float* m2,
                      __nv_bfloat16* lp, const AdamW h, const int* skip_flag, uint32_t epoch, int* status) {
  uint32_t done_base;
  const bool ok = collective_begin(P, epoch, status, done_base);
  if (ok && !(skip_flag && *skip_flag)) {
    const long lo = grad_off + shard * 2 * P.rank;
    for (long i = ((long)blockIdx.x * kThreads + threadIdx.x) * 8; i < shard;
         i += (long)gridDim.x * kThreads * 8) {
      float g[8];
      reduce16<true, MC>(P, lo + i * 2, g);
      float4 w0 = *reinterpret_cast<float4*>(master + i), w1 = *reinterpret_cast<float4*>(master + i + 4);
      float4 a0 = *reinterpret_cast<float4*>(m1 + i), a1 = *reinterpret_cast<float4*>(m1 + i + 4);
      float4 b0 = *reinterpret_cast<float4*>(m2 + i), b1 = *reinterpret_cast<float4*>(m2 + i + 4);
      float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gr = g[j] * h.mul;
        w[j] *= 1.f - h.lr * h.wd;
        a[j] = h.beta1 * a[j] + (1.f - h.beta1) * gr;
        b[j] = h.beta2 * b[j] + (1.f - h.beta2) * gr * gr;
        w[j] -= (h.lr / h.bc1) * a[j] / (sqrtf(b[j] / h.bc2) + h.eps);
      }
      *reinterpret_cast<float4*>(master + i) = make_float4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<float4*>(master + i + 4) = make_float4(w[4], w[5], w[6], w[7]);
      *reinterpret_cast<float4*>(m1 + i) = make_float4(a[0], a[1], a[2], a[3]);
      *reinterpret_cast<float4*>(m1 + i + 4) = make_float4(a[4], a[5], a[6], a[7]);
      *reinterpret_cast<float4*>(m2 + i) = make_float4(b[0], b[1], b[2], b[3]);
      *reinterpret_cast<float4*>(m2 + i + 4) = make_float4(b[4], b[5], b[6], b[7]);
      const uint4 packed = pack_bf16x8(w);
      if (lp) *reinterpret_cast<uint4*>(lp + i) = packed;
    }
  }
  collective_end(P, epoch, 0, status, done_base);
}

// First phase of LAMB on a sharded unit, fused with the gradient reduce-scatter: rank r sums its shard
// of every peer's flat gradient, updates the moments and writes the per-element update
//   c = (m / bc1) / (sqrt(v / bc2) + eps) + wd * w
// into `upd`, and adds this shard's share of sum(w^2) and sum(c^2) of every tensor to
// norms[2 * tensor id + {0, 1}].  A shard holds whole or partial tensors back to back; seg_start
// [nseg + 1] are their boundaries inside the shard (multiples of 8 elements, the tensors are laid out
// on 64-element boundaries) and seg_gid[nseg] their ids.  The second phase (trust ratio per tensor
// from the norms summed over ranks, then w -= lr * trust * c) runs once all units have finished
// this one (lamb.rs:200-280 of the reference does both per parameter on unsharded tensors).
template <bool MC>
__global__ void __launch_bounds__(kThreads)
fused_rs_lamb1_kernel(const Peers P, long grad_off, long shard, const float* __restrict__ master, float* m1, float* m2,
                      float* upd, const long* __restrict__ seg_start, const int* __restrict__ seg_gid, int nseg,
                      float* norms, const AdamW h, const int* skip_flag, uint32_t epoch, int* status) {
  uint32_t done_base;
  const bool ok = collective_begin(P, epoch, status, done_base);
  if (ok && !(skip_flag && *skip_flag)) {
    const long lo = grad_off + shard * 2 * P.rank;
    for (long i0 = (long)blockIdx.x * kThreads * 8; i0 < shard; i0 += (long)gridDim.x * kThreads * 8) {
      const long i = i0 + (long)threadIdx.x * 8;
      float sw = 0.f, sc = 0.f;
      int seg = -1;
      if (i < shard) {
        float g[8];
        reduce16<true, MC>(P, lo + i * 2, g);
        const float4 w0 = *reinterpret_cast<const float4*>(master + i), w1 = *reinterpret_cast<const float4*>(master + i + 4);
        float4 a0 = *reinterpret_cast<float4*>(m1 + i), a1 = *reinterpret_cast<float4*>(m1 + i + 4);
        float4 b0 = *reinterpret_cast<float4*>(m2 + i), b1 = *reinterpret_cast<float4*>(m2 + i + 4);
        const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        float c[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gr = g[j] * h.mul;
          a[j] = h.beta1 * a[j] + (1.f - h.beta1) * gr;
          b[j] = h.beta2 * b[j] + (1.f - h.beta2) * gr * gr;
          c[j] = (a[j] / h.bc1) / (sqrtf(b[j] / h.bc2) + h.eps) + h.wd * w[j];
          sw += w[j] * w[j];
          sc += c[j] * c[j];
        }
        *reinterpret_cast<float4*>(m1 + i) = make_float4(a[0], a[1], a[2], a[3]);
        *reinterpret_cast<float4*>(m1 + i + 4) = make_float4(a[4], a[5], a[6], a[7]);
        *reinterpret_cast<float4*>(m2 + i) = make_float4(b[0], b[1], b[2], b[3]);
        *reinterpret_cast<float4*>(m2 + i + 4) = make_float4(b[4], b[5], b[6], b[7]);
        *reinterpret_cast<float4*>(upd + i) = make_float4(c[0], c[1], c[2], c[3]);
        *reinterpret_cast<float4*>(upd + i + 4) = make_float4(c[4], c[5], c[6], c[7]);
        // the tensor these 8 elements belong to (a handful of tensors per shard: a linear scan)
        for (int k = 0; k < nseg; ++k)
          if (i >= seg_start[k] && i < seg_start[k + 1]) { seg = k; break; }
      }
      // one pair of atomics per warp when the whole warp sits in one tensor, else per lane
      const int seg0 = __shfl_sync(0xffffffffu, seg, 0);
      if (__all_sync(0xffffffffu, seg == seg0)) {
        sw = warp_sum(sw);
        sc = warp_sum(sc);
        if ((threadIdx.x & 31) == 0 && seg0 >= 0) {
          atomicAdd(norms + 2 * seg_gid[seg0], sw);
          atomicAdd(norms + 2 * seg_gid[seg0] + 1, sc);
        }
      } else if (seg >= 0) {
        atomicAdd(norms + 2 * seg_gid[seg], sw);
        atomicAdd(norms + 2 * seg_gid[seg] + 1, sc);
      }
    }
  }
  collective_end(P, epoch, 0, status, done_base);
}

// Every launch on one communicator uses the same grid (the per-GPU completion counter advances by
// exactly `grid` per epoch); kernels are grid-stride, so any size is correct.
int checked_grid(int grid) {
  int sms = axh::sm_count();
  if (grid < 1) grid = 1;
  if (grid > sms) grid = sms;       // all blocks must be resident together
  return grid;
}

Peers make_peers(void* const* bufs, void* const* sigs, void* mc, int rank, int world) {
  Peers P;
  for (int i = 0; i < kMaxRanks; ++i) {
    P.buf[i] = i < world && bufs ? bufs[i] : nullptr;
    P.sig[i] = i < world && sigs ? (uint32_t*)sigs[i] : nullptr;
  }
  P.mc_buf = mc;
  P.rank = rank;
  P.world = world;
  return P;
}

}  // namespace

// Number of 32-bit signal slots a communicator must provide per rank (zero-initialised once).
AX_API int ax_comm_signal_slots() { return 2 * axc::kMaxRanks + 4 + 2 * axc::kMaxRanks; }

// out = mul * sum over ranks of x (`bytes` of bf16 (dtype 1) or fp32 (dtype 0), a multiple of 16, at most
// `slot_bytes`); x and out may be the same ordinary device buffer.  `bufs` are the ranks' staging buffers of
// 2 * world * slot_bytes bytes; `epoch_dev` is this communicator's call counter on the device (one per
// communicator, used for nothing else).  Every rank must make the same sequence of calls.
AX_API int ax_oneshot_allreduce(int dtype, void* const* bufs, void* const* sigs, void* mc_buf, int rank, int world,
                                const void* x, void* out, long bytes, long slot_bytes, float mul, unsigned* epoch_dev,
                                int* status, cudaStream_t stream) {
  if (world < 1 || world > axc::kMaxRanks || bytes <= 0 || bytes % 16 || slot_bytes % 16 || bytes > slot_bytes ||
      epoch_dev == nullptr)
    return -1;
  if (((uintptr_t)x | (uintptr_t)out) & 15) return -1;
  Peers P = make_peers(bufs, sigs, mc_buf, rank, world);
  const auto* xi = (const uint8_t*)x;
  auto* xo = (uint8_t*)out;
  if (dtype == 1) {
    if (mc_buf) oneshot_allreduce_kernel<true, true><<<1, kOneShotThreads, 0, stream>>>(P, xi, xo, bytes, slot_bytes, mul, epoch_dev, status);
    else oneshot_allreduce_kernel<true, false><<<1, kOneShotThreads, 0, stream>>>(P, xi, xo, bytes, slot_bytes, mul, epoch_dev, status);
  } else {
    if (mc_buf) oneshot_allreduce_kernel<false, true><<<1, kOneShotThreads, 0, stream>>>(P, xi, xo, bytes, slot_bytes, mul, epoch_dev, status);
    else oneshot_allreduce_kernel<false, false><<<1, kOneShotThreads, 0, stream>>>(P, xi, xo, bytes, slot_bytes, mul, epoch_dev, status);
  }
  return (int)cudaGetLastError();
}

// In-place mean all-reduce of `n` elements (dtype: 0 fp32, 1 bf16) located at byte offset
// `base_off` of every rank's symmetric buffer.  n * elsize must be a multiple of 16 * world.
// `epoch` must increase by one per call on this communicator (all ranks use the same value).
// `epoch_dev` (optional): device word that replaces `epoch` (see the kernel); a communicator must use one
// of the two consistently.
AX_API int ax_fused_allreduce(int dtype, void* const* bufs, void* const* sigs, void* mc_buf, int rank,
                              int world, long base_off, long n, const float* inv_scale, int* found_inf,
                              unsigned epoch, unsigned* epoch_dev, int grid_blocks, int* status, cudaStream_t stream) {
  if (world < 1 || world > axc::kMaxRanks) return -1;
  const int esz = dtype == 1 ? 2 : 4;
  if ((n * esz) % (16L * world) || (base_off % 16)) return -1;
  Peers P = make_peers(bufs, sigs, mc_buf, rank, world);
  const int grid = checked_grid(grid_blocks);
  const float mul = 1.f / world;
  if (dtype == 1) {
    if (mc_buf) fused_allreduce_kernel<true, true><<<grid, kThreads, 0, stream>>>(P, base_off, n, mul, inv_scale, found_inf, epoch, epoch_dev, status);
    else fused_allreduce_kernel<true, false><<<grid, kThreads, 0, stream>>>(P, base_off, n, mul, inv_scale, found_inf, epoch, epoch_dev, status);
  } else {
    if (mc_buf) fused_allreduce_kernel<false, true><<<grid, kThreads, 0, stream>>>(P, base_off, n, mul, inv_scale, found_inf, epoch, epoch_dev, status);
    else fused_allreduce_kernel<false, false><<<grid, kThreads, 0, stream>>>(P, base_off, n, mul, inv_scale, found_inf, epoch, epoch_dev, status);
  }
  return (int)cudaGetLastError();
}

// hyper: float[7] = lr, beta1, beta2, eps, wd, bc1 (1-beta1^t), bc2 (1-beta2^t).
// `shard` (elements per rank) must be a multiple of 8; grad_off is a byte offset.
AX_API int ax_fused_rs_adamw(void* const* grad_bufs, void* const* sigs, void* grad_mc, int rank,
                             int world, long grad_off, long shard, float* master, float* m1, float* m2,
                             void* lp, const float* hyper, const int* skip_flag, unsigned epoch, int grid_blocks,
                             int* status, cudaStream_t stream) {
  if (world < 1 || world > axc::kMaxRanks || shard % 8 || grad_off % 16) return -1;
  Peers P = make_peers(grad_bufs, sigs, grad_mc, rank, world);
  AdamW h{hyper[0], hyper[1], hyper[2], hyper[3], hyper[4], hyper[5], hyper[6], 1.f / world};
  const int grid = checked_grid(grid_blocks);
  if (grad_mc)
    fused_rs_adamw_kernel<true><<<grid, kThreads, 0, stream>>>(P, grad_off, shard, master, m1, m2, (__nv_bfloat16*)lp, h, skip_flag, epoch, status);
  else
    fused_rs_adamw_kernel<false><<<grid, kThreads, 0, stream>>>(P, grad_off, shard, master, m1, m2, (__nv_bfloat16*)lp, h, skip_flag, epoch, status);
  return (int)cudaGetLastError();
}

// First LAMB phase fused with the reduce-scatter of a unit's flat gradient (see the kernel).
// hyper: float[7] as for ax_fused_rs_adamw (lr is not used here).  `upd` [shard] fp32 receives the
// per-element update, `norms` [num_tensors][2] fp32 (zeroed by the caller once per step) the sums.
AX_API int ax_fused_rs_lamb1(void* const* grad_bufs, void* const* sigs, void* grad_mc, int rank, int world,
                             long grad_off, long shard, const float* master, float* m1, float* m2, float* upd,
                             const long* seg_start, const int* seg_gid, int nseg, float* norms,
                             const float* hyper, const int* skip_flag, unsigned epoch, int grid_blocks,
                             int* status, cudaStream_t stream) {
  if (world < 1 || world > axc::kMaxRanks || shard % 8 || grad_off % 16 || nseg < 0) return -1;
  Peers P = make_peers(grad_bufs, sigs, grad_mc, rank, world);
  AdamW h{hyper[0], hyper[1], hyper[2], hyper[3], hyper[4], hyper[5], hyper[6], 1.f / world};
  const int grid = checked_grid(grid_blocks);
  if (grad_mc)
    fused_rs_lamb1_kernel<true><<<grid, kThreads, 0, stream>>>(P, grad_off, shard, master, m1, m2, upd, seg_start, seg_gid, nseg, norms, h, skip_flag, epoch, status);
  else
    fused_rs_lamb1_kernel<false><<<grid, kThreads, 0, stream>>>(P, grad_off, shard, master, m1, m2, upd, seg_start, seg_gid, nseg, norms, h, skip_flag, epoch, status);
  return (int)cudaGetLastError();
}
