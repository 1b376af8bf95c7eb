// LayerNorm / RMSNorm forward and backward, bf16 or fp32 activations, fp32 statistics.
// One warp per row.  bf16 rows up to 8192 wide are read once and kept in registers (packed) between
// the statistics and the normalisation; other rows are read twice (the second read is served by
// L1/L2), so HBM traffic is one read of x and one write of y either way.  The optional residual input fuses `h = x + r` (h is written
// out as the new residual stream) with the normalisation of h.
//
// Backward: per-row dx in one pass; weight/bias gradients are accumulated per CTA in shared
// memory, written as per-CTA partials to a scratch buffer [grid, 2, D] and summed by a second
// kernel (deterministic, no global atomics).
//
// Parity: crates/axonml-nn/src/layers/norm.rs:447-482 (LayerNorm), crates/axonml-llm/src/llama.rs:158-187
// (RMSNorm), and the WGSL layer-norm shader arithmetic (wgpu_backend.rs:1318-1361).
#include "common.cuh"

namespace {
using namespace ax;

template <typename T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
           d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
    u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  static __device__ __forceinline__ void round_trip(float (&v)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
  }
};
template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  static __device__ __forceinline__ void round_trip(float (&)[8]) {}
};

constexpr int kWarpsPerCta = 8;

// x, res, y, hout: [rows, D] (row stride D); w, b: [D] of type WT; mean/rstd: [rows] fp32.
template <typename T, typename WT, bool RMS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const WT* __restrict__ w,
                const WT* __restrict__ b, T* __restrict__ y, T* __restrict__ hout,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int D,
                float eps) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (long row = (long)blockIdx.x * kWarpsPerCta + warp; row < rows;
       row += (long)gridDim.x * kWarpsPerCta) {
    const T* xr = x + row * D;
    const T* rr = res ? res + row * D : nullptr;
    T* hr = hout ? hout + row * D : nullptr;
    float s = 0.f, ss = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      float v[8];
      Vec8<T>::load(xr + c, v);
      if (rr) {
        float r[8];
        Vec8<T>::load(rr + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += r[j];
        if (hr) {
          // round to the storage type so that the statistics match what backward re-reads
          Vec8<T>::store(hr + c, v);
          Vec8<T>::load(hr + c, v);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[j]; ss += v[j] * v[j]; }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    float mean = RMS ? 0.f : s / D;
    float var = RMS ? ss / D : fmaxf(ss / D - mean * mean, 0.f);
    float rstd = rsqrtf(var + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    const T* src = (rr && hr) ? hr : xr;
    T* yr = y + row * D;
    for (int c = lane * 8; c < D; c += 256) {
      float v[8], wv[8], bv[8];
      Vec8<T>::load(src + c, v);
      if (rr && !hr) {
        float r[8];
        Vec8<T>::load(rr + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += r[j];
      }
      Vec8<WT>::load(w + c, wv);
      if (b) Vec8<WT>::load(b + c, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float o = (v[j] - mean) * rstd * wv[j];
        v[j] = b ? o + bv[j] : o;
      }
      Vec8<T>::store(yr + c, v);
    }
  }
}

// Many rows of bf16 with D <= 256 * NV: one warp per row, the row read ONCE and kept in registers as
// the packed bf16 it arrived as (4 registers per 8 values, so even D = 8192 fits), all loads of a
// row in flight together; the statistics and the normalisation both unpack from the registers.
// For NV <= 8 the weight (and bias) vectors of the lane's columns are loaded once per warp and
// reused for every row the warp handles.
template <typename WT, bool RMS, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
norm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res, const WT* __restrict__ w,
                    const WT* __restrict__ b, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ hout,
                    float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int D, float eps) {
  using T = __nv_bfloat16;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  constexpr bool kKeepW = NV <= 8;
  float wreg[kKeepW ? NV : 1][8], breg[kKeepW ? NV : 1][8];
  if (kKeepW) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < D) {
        Vec8<WT>::load(w + c, wreg[i]);
        if (b) Vec8<WT>::load(b + c, breg[i]);
      }
    }
  }
  for (long row = (long)blockIdx.x * kWarpsPerCta + warp; row < rows; row += (long)gridDim.x * kWarpsPerCta) {
    const T* xr = x + row * D;
    const T* rr = res ? res + row * D : nullptr;
    T* hr = hout ? hout + row * D : nullptr;
    uint4 xv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < D) xv[i] = *reinterpret_cast<const uint4*>(xr + c);
    }
    if (rr) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane * 8 + i * 256;
        if (c < D) {
          const uint4 rv = *reinterpret_cast<const uint4*>(rr + c);
          const float2 a0 = unpack_bf16x2(xv[i].x), a1 = unpack_bf16x2(xv[i].y), a2 = unpack_bf16x2(xv[i].z), a3 = unpack_bf16x2(xv[i].w);
          const float2 r0 = unpack_bf16x2(rv.x), r1 = unpack_bf16x2(rv.y), r2 = unpack_bf16x2(rv.z), r3 = unpack_bf16x2(rv.w);
          // h = x + r rounded to the storage type: the statistics are those of what backward re-reads
          xv[i].x = pack_bf16x2(a0.x + r0.x, a0.y + r0.y); xv[i].y = pack_bf16x2(a1.x + r1.x, a1.y + r1.y);
          xv[i].z = pack_bf16x2(a2.x + r2.x, a2.y + r2.y); xv[i].w = pack_bf16x2(a3.x + r3.x, a3.y + r3.y);
          if (hr) *reinterpret_cast<uint4*>(hr + c) = xv[i];
        }
      }
    }
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < D) {
        const float2 a0 = unpack_bf16x2(xv[i].x), a1 = unpack_bf16x2(xv[i].y), a2 = unpack_bf16x2(xv[i].z), a3 = unpack_bf16x2(xv[i].w);
        s += (a0.x + a0.y) + (a1.x + a1.y) + (a2.x + a2.y) + (a3.x + a3.y);
        ss += (a0.x * a0.x + a0.y * a0.y) + (a1.x * a1.x + a1.y * a1.y) + (a2.x * a2.x + a2.y * a2.y) + (a3.x * a3.x + a3.y * a3.y);
      }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    const float mean = RMS ? 0.f : s / D;
    const float var = RMS ? ss / D : fmaxf(ss / D - mean * mean, 0.f);
    const float rstd = rsqrtf(var + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    T* yr = y + row * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < D) {
        float v[8], wv[8], bv[8];
        const float2 a0 = unpack_bf16x2(xv[i].x), a1 = unpack_bf16x2(xv[i].y), a2 = unpack_bf16x2(xv[i].z), a3 = unpack_bf16x2(xv[i].w);
        v[0] = a0.x; v[1] = a0.y; v[2] = a1.x; v[3] = a1.y; v[4] = a2.x; v[5] = a2.y; v[6] = a3.x; v[7] = a3.y;
        if (!kKeepW) {
          Vec8<WT>::load(w + c, wv);
          if (b) Vec8<WT>::load(b + c, bv);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float o = (v[j] - mean) * rstd * (kKeepW ? wreg[i][j] : wv[j]);
          v[j] = b ? o + (kKeepW ? breg[i][j] : bv[j]) : o;
        }
        Vec8<T>::store(yr + c, v);
      }
    }
  }
}

template <typename WT, int NV>
int launch_fwd_reg(bool rms, const void* x, const void* res, const void* w, const void* b, void* y, void* hout,
                   float* mean, float* rstd, int rows, int D, float eps, cudaStream_t stream) {
  int grid = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  // One resident wave: a warp then walks over several rows with the weights it loaded once.  (With eight
  // CTAs per SM in the grid a [8192, 2048] call gave every warp ONE row and 8 KB of weights to load for
  // it: 60 us for 134 MB in the GPT-1.3B step.)
  int occ = 1;
  if (rms) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, norm_fwd_reg_kernel<WT, true, NV>, kWarpsPerCta * 32, 0);
  else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, norm_fwd_reg_kernel<WT, false, NV>, kWarpsPerCta * 32, 0);
  const int cap = axh::sm_count() * (occ < 1 ? 1 : occ);
  if (grid > cap) grid = cap;
  using T = __nv_bfloat16;
  if (rms)
    norm_fwd_reg_kernel<WT, true, NV><<<grid, kWarpsPerCta * 32, 0, stream>>>((const T*)x, (const T*)res, (const WT*)w,
                                                                         (const WT*)b, (T*)y, (T*)hout, mean, rstd, rows, D, eps);
  else
    norm_fwd_reg_kernel<WT, false, NV><<<grid, kWarpsPerCta * 32, 0, stream>>>((const T*)x, (const T*)res, (const WT*)w,
                                                                          (const WT*)b, (T*)y, (T*)hout, mean, rstd, rows, D, eps);
  return (int)cudaGetLastError();
}

// Few rows (decode steps, small batches): one CTA per row, the row held in registers between
// the statistics and the normalisation, so the row is read once and all its loads are in flight
// together.  (With many rows the warp-per-row kernel is faster: 3.8 TB/s against 2.1 TB/s at
// [65536, 4096].)  D <= kWarpsPerCta * 32 * 8 * kBlockVecs.
constexpr int kBlockVecs = 8;
template <typename T, typename WT, bool RMS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
norm_fwd_block_kernel(const T* __restrict__ x, const T* __restrict__ res, const WT* __restrict__ w,
                      const WT* __restrict__ b, T* __restrict__ y, T* __restrict__ hout,
                      float* __restrict__ mean_out, float* __restrict__ rstd_out, int D, float eps) {
  constexpr int kStep = kWarpsPerCta * 32 * 8;
  __shared__ float red[2][kWarpsPerCta];
  const long row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* xr = x + row * D;
  const T* rr = res ? res + row * D : nullptr;
  T* hr = hout ? hout + row * D : nullptr;
  float v[kBlockVecs][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < kBlockVecs; ++i) {
    const int c = threadIdx.x * 8 + i * kStep;
    if (c < D) {
      Vec8<T>::load(xr + c, v[i]);
      if (rr) {
        float r[8];
        Vec8<T>::load(rr + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        if (hr) {
          Vec8<T>::store(hr + c, v[i]);
          Vec8<T>::round_trip(v[i]);      // statistics of the stored (rounded) values
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[i][j]; ss += v[i][j] * v[i][j]; }
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  if (lane == 0) { red[0][warp] = s; red[1][warp] = ss; }
  __syncthreads();
  s = 0.f; ss = 0.f;
#pragma unroll
  for (int i = 0; i < kWarpsPerCta; ++i) { s += red[0][i]; ss += red[1][i]; }
  const float mean = RMS ? 0.f : s / D;
  const float var = RMS ? ss / D : fmaxf(ss / D - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  T* yr = y + row * D;
#pragma unroll
  for (int i = 0; i < kBlockVecs; ++i) {
    const int c = threadIdx.x * 8 + i * kStep;
    if (c < D) {
      float wv[8], bv[8];
      Vec8<WT>::load(w + c, wv);
      if (b) Vec8<WT>::load(b + c, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float o = (v[i][j] - mean) * rstd * wv[j];
        v[i][j] = b ? o + bv[j] : o;
      }
      Vec8<T>::store(yr + c, v[i]);
    }
  }
}

// dx per row; per-CTA partial sums of dw (and db) into `partial` [gridDim.x, 2, D].
// If `dres_in` is given it is added to dx (gradient arriving through the residual stream).
template <typename T, typename WT, bool RMS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const WT* __restrict__ w,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                const T* __restrict__ dres_in, T* __restrict__ dx, float* __restrict__ partial,
                int rows, int D) {
  // [2][Dp], Dp = D rounded up to 256.  Column (b*256 + l*8 + j) lives at b*256 + j*32 + l so
  // that the 32 lanes of a warp always hit 32 different banks.
  extern __shared__ float sacc[];
  const int Dp = ((D + 255) / 256) * 256;
  float* sdw = sacc;
  float* sdb = sacc + Dp;
  for (int i = threadIdx.x; i < 2 * Dp; i += blockDim.x) sacc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (long row = (long)blockIdx.x * kWarpsPerCta + warp; row < rows;
       row += (long)gridDim.x * kWarpsPerCta) {
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;  // sum(dy*w), sum(dy*w*xhat)
    for (int c = lane * 8; c < D; c += 256) {
      float xv[8], gv[8], wv[8];
      Vec8<T>::load(xr + c, xv);
      Vec8<T>::load(dyr + c, gv);
      Vec8<WT>::load(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float xh = (xv[j] - mean) * rstd;
        float gw = gv[j] * wv[j];
        s1 += gw;
        s2 += gw * xh;
        const int slot = (c - lane * 8) + j * 32 + lane;
        atomicAdd(&sdw[slot], gv[j] * xh);
        if (!RMS) atomicAdd(&sdb[slot], gv[j]);
      }
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    if (RMS) s1 = 0.f;
    T* dxr = dx + row * D;
    const T* drr = dres_in ? dres_in + row * D : nullptr;
    for (int c = lane * 8; c < D; c += 256) {
      float xv[8], gv[8], wv[8], o[8];
      Vec8<T>::load(xr + c, xv);
      Vec8<T>::load(dyr + c, gv);
      Vec8<WT>::load(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float xh = (xv[j] - mean) * rstd;
        o[j] = rstd * (gv[j] * wv[j] - s1 - xh * s2);
      }
      if (drr) {
        float r[8];
        Vec8<T>::load(drr + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      Vec8<T>::store(dxr + c, o);
    }
  }
  __syncthreads();
  float* out = partial + (long)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * Dp; i += blockDim.x) {
    const int which = i / Dp, pos = i - which * Dp;
    const int rem = pos & 255;
    const int col = (pos - rem) + (rem & 31) * 8 + (rem >> 5);
    if (col < D) out[which * D + col] = sacc[i];
  }
}

// Same contract as norm_bwd_kernel for D == ITERS * 256: the weight- and bias-gradient partial sums
// of the columns a lane owns stay in registers over all rows of its warp (no shared-memory atomics
// in the row loop) and the warps of a CTA are combined once at the end.
template <typename T, typename WT, bool RMS, int ITERS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
norm_bwd_reg_kernel(const T* __restrict__ dy, const T* __restrict__ x, const WT* __restrict__ w,
                    const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                    const T* __restrict__ dres_in, T* __restrict__ dx, float* __restrict__ partial, int rows) {
  constexpr int D = ITERS * 256;
  extern __shared__ float sacc[];            // [RMS ? 1 : 2][D]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float aw[ITERS][8];
  float ab[RMS ? 1 : ITERS][8];
#pragma unroll
  for (int i = 0; i < ITERS; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { aw[i][j] = 0.f; if (!RMS) ab[i][j] = 0.f; }
  for (long row = (long)blockIdx.x * kWarpsPerCta + warp; row < rows; row += (long)gridDim.x * kWarpsPerCta) {
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      float xv[8], gv[8], wv[8];
      Vec8<T>::load(xr + i * 256 + lane * 8, xv);
      Vec8<T>::load(dyr + i * 256 + lane * 8, gv);
      Vec8<WT>::load(w + i * 256 + lane * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (xv[j] - mean) * rstd;
        const float gw = gv[j] * wv[j];
        s1 += gw;
        s2 += gw * xh;
        aw[i][j] += gv[j] * xh;
        if (!RMS) ab[i][j] += gv[j];
      }
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    if (RMS) s1 = 0.f;
    T* dxr = dx + row * D;
    const T* drr = dres_in ? dres_in + row * D : nullptr;
    // second pass over the row (4-16 KB, still in L1): the accumulators own the registers
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      float xv[8], gv[8], wv[8], o[8];
      Vec8<T>::load(xr + i * 256 + lane * 8, xv);
      Vec8<T>::load(dyr + i * 256 + lane * 8, gv);
      Vec8<WT>::load(w + i * 256 + lane * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (gv[j] * wv[j] - s1 - (xv[j] - mean) * rstd * s2);
      if (drr) {
        float r[8];
        Vec8<T>::load(drr + i * 256 + lane * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      Vec8<T>::store(dxr + i * 256 + lane * 8, o);
    }
  }
  for (int wi = 0; wi < kWarpsPerCta; ++wi) {
    if (warp == wi) {
#pragma unroll
      for (int i = 0; i < ITERS; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int d = i * 256 + j * 32 + lane;        // conflict-free slot of column i*256 + lane*8 + j
          if (wi == 0) { sacc[d] = aw[i][j]; if (!RMS) sacc[D + d] = ab[i][j]; }
          else { sacc[d] += aw[i][j]; if (!RMS) sacc[D + d] += ab[i][j]; }
        }
    }
    __syncthreads();
  }
  float* out = partial + (long)blockIdx.x * 2 * D;
  for (int t = threadIdx.x; t < D; t += blockDim.x) {
    const int rem = t & 255;
    const int col = (t - rem) + (rem & 31) * 8 + (rem >> 5);
    out[col] = sacc[t];
    if (!RMS) out[D + col] = sacc[D + t];
  }
}

// dw[d] = sum_g partial[g,0,d]; db[d] = sum_g partial[g,1,d].  Block = 32 columns x 32 group
// lanes: each thread sums groups g = ty, ty+32, ..., then the 32 partials of a column are combined
// through shared memory.
template <typename WT>
__global__ void norm_bwd_reduce_kernel(const float* __restrict__ partial, WT* __restrict__ dw,
                                       WT* __restrict__ db, int groups, int D) {
  __shared__ float sa[32][33], sb[32][33];
  const int d = blockIdx.x * 32 + threadIdx.x;
  float a = 0.f, b = 0.f;
  if (d < D) {
    for (int g = threadIdx.y; g < groups; g += 32) {
      a += partial[(long)g * 2 * D + d];
      if (db) b += partial[(long)g * 2 * D + D + d];
    }
  }
  sa[threadIdx.y][threadIdx.x] = a;
  sb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && d < D) {
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) { ta += sa[j][threadIdx.x]; tb += sb[j][threadIdx.x]; }
    if (dw) dw[d] = (WT)ta;
    if (db) db[d] = (WT)tb;
  }
}

template <typename T, typename WT>
int launch_fwd(bool rms, const void* x, const void* res, const void* w, const void* b, void* y,
               void* hout, float* mean, float* rstd, int rows, int D, float eps,
               cudaStream_t stream) {
  if (rows <= axh::sm_count() * 4 && D >= 1024 && D <= kWarpsPerCta * 32 * 8 * kBlockVecs) {
    if (rms)
      norm_fwd_block_kernel<T, WT, true><<<rows, kWarpsPerCta * 32, 0, stream>>>(
          (const T*)x, (const T*)res, (const WT*)w, (const WT*)b, (T*)y, (T*)hout, mean, rstd, D, eps);
    else
      norm_fwd_block_kernel<T, WT, false><<<rows, kWarpsPerCta * 32, 0, stream>>>(
          (const T*)x, (const T*)res, (const WT*)w, (const WT*)b, (T*)y, (T*)hout, mean, rstd, D, eps);
    return (int)cudaGetLastError();
  }
  if (sizeof(T) == 2 && D <= 8192 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)res | (uintptr_t)hout | (uintptr_t)w | (uintptr_t)b) & 15) == 0) {
    // bf16 rows that fit the register file: single pass
    if (D <= 1024) return launch_fwd_reg<WT, 4>(rms, x, res, w, b, y, hout, mean, rstd, rows, D, eps, stream);
    if (D <= 2048) return launch_fwd_reg<WT, 8>(rms, x, res, w, b, y, hout, mean, rstd, rows, D, eps, stream);
    if (D <= 4096) return launch_fwd_reg<WT, 16>(rms, x, res, w, b, y, hout, mean, rstd, rows, D, eps, stream);
    return launch_fwd_reg<WT, 32>(rms, x, res, w, b, y, hout, mean, rstd, rows, D, eps, stream);
  }
  int grid = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  int cap = axh::sm_count() * 8;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  if (rms)
    norm_fwd_kernel<T, WT, true><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        (const T*)x, (const T*)res, (const WT*)w, (const WT*)b, (T*)y, (T*)hout, mean, rstd, rows,
        D, eps);
  else
    norm_fwd_kernel<T, WT, false><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        (const T*)x, (const T*)res, (const WT*)w, (const WT*)b, (T*)y, (T*)hout, mean, rstd, rows,
        D, eps);
  return (int)cudaGetLastError();
}

template <typename T, typename WT>
int launch_bwd(bool rms, const void* dy, const void* x, const void* w, const float* mean,
               const float* rstd, const void* dres, void* dx, void* dw, void* db, float* scratch,
               int groups, int rows, int D, cudaStream_t stream) {
  // register-accumulating variant for the common widths (accumulators must fit the register file)
  bool done = false;
#define AX_NORM_BWD_REG(RMSV, IT)                                                                              \
  if (!done && rms == RMSV && D == IT * 256) {                                                                 \
    norm_bwd_reg_kernel<T, WT, RMSV, IT><<<groups, kWarpsPerCta * 32, (RMSV ? 1 : 2) * D * sizeof(float), stream>>>( \
        (const T*)dy, (const T*)x, (const WT*)w, mean, rstd, (const T*)dres, (T*)dx, scratch, rows);           \
    done = true;                                                                                               \
  }
  AX_NORM_BWD_REG(false, 1) AX_NORM_BWD_REG(false, 2) AX_NORM_BWD_REG(false, 3) AX_NORM_BWD_REG(false, 4)
  AX_NORM_BWD_REG(false, 8)
  AX_NORM_BWD_REG(true, 1) AX_NORM_BWD_REG(true, 2) AX_NORM_BWD_REG(true, 4) AX_NORM_BWD_REG(true, 8)
#undef AX_NORM_BWD_REG
  if (done) {
    cudaError_t e0 = cudaGetLastError();
    if (e0 != cudaSuccess) return (int)e0;
    norm_bwd_reduce_kernel<WT><<<(D + 31) / 32, dim3(32, 32), 0, stream>>>(scratch, (WT*)dw, rms ? nullptr : (WT*)db,
                                                                     groups, D);
    return (int)cudaGetLastError();
  }
  size_t smem = (size_t)2 * (((D + 255) / 256) * 256) * sizeof(float);
  if (rms) {
    auto k = norm_bwd_kernel<T, WT, true>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<groups, kWarpsPerCta * 32, smem, stream>>>((const T*)dy, (const T*)x, (const WT*)w, mean,
                                                   rstd, (const T*)dres, (T*)dx, scratch, rows, D);
  } else {
    auto k = norm_bwd_kernel<T, WT, false>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<groups, kWarpsPerCta * 32, smem, stream>>>((const T*)dy, (const T*)x, (const WT*)w, mean,
                                                   rstd, (const T*)dres, (T*)dx, scratch, rows, D);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  norm_bwd_reduce_kernel<WT><<<(D + 31) / 32, dim3(32, 32), 0, stream>>>(scratch, (WT*)dw,
                                                                   rms ? nullptr : (WT*)db, groups, D);
  return (int)cudaGetLastError();
}

}  // namespace

// dtype codes: 0 = fp32, 1 = bf16.  D must be a multiple of 8.
AX_API int ax_norm_fwd(int rms, int act_dtype, int w_dtype, const void* x, const void* res,
                       const void* w, const void* b, void* y, void* hout, float* mean, float* rstd,
                       int rows, int D, float eps, cudaStream_t stream) {
  if (D % 8 != 0 || rows <= 0) return -1;
  if (act_dtype == 1 && w_dtype == 1)
    return launch_fwd<__nv_bfloat16, __nv_bfloat16>(rms, x, res, w, b, y, hout, mean, rstd, rows, D, eps, stream);
  if (act_dtype == 1 && w_dtype == 0)
    return launch_fwd<__nv_bfloat16, float>(rms, x, res, w, b, y, hout, mean, rstd, rows, D, eps, stream);
  if (act_dtype == 0 && w_dtype == 0)
    return launch_fwd<float, float>(rms, x, res, w, b, y, hout, mean, rstd, rows, D, eps, stream);
  return -1;
}

// Number of per-CTA partial slots the backward uses for `rows` rows; scratch must hold
// groups * 2 * D floats.
AX_API int ax_norm_bwd_groups(int rows) {
  int g = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  int cap = axh::sm_count() * 2;
  if (g > cap) g = cap;
  return g < 1 ? 1 : g;
}

AX_API int ax_norm_bwd(int rms, int act_dtype, int w_dtype, const void* dy, const void* x,
                       const void* w, const float* mean, const float* rstd, const void* dres,
                       void* dx, void* dw, void* db, float* scratch, int groups, int rows, int D,
                       cudaStream_t stream) {
  if (D % 8 != 0 || rows <= 0 || groups <= 0) return -1;
  if (act_dtype == 1 && w_dtype == 1)
    return launch_bwd<__nv_bfloat16, __nv_bfloat16>(rms, dy, x, w, mean, rstd, dres, dx, dw, db, scratch, groups, rows, D, stream);
  if (act_dtype == 1 && w_dtype == 0)
    return launch_bwd<__nv_bfloat16, float>(rms, dy, x, w, mean, rstd, dres, dx, dw, db, scratch, groups, rows, D, stream);
  if (act_dtype == 0 && w_dtype == 0)
    return launch_bwd<float, float>(rms, dy, x, w, mean, rstd, dres, dx, dw, db, scratch, groups, rows, D, stream);
  return -1;
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant of the norm backward (declared in axonml_noalloc.h).
//
// Some callers cannot allocate device memory: code running inside a CUDA-graph capture or a
// latency-critical serving loop where cudaMalloc would synchronise the device, plugins that are
// handed a fixed arena by their host application, and processes whose memory pool is owned by
// another runtime.  For them the per-CTA partial sums live in a fixed array inside this library
// instead of a caller-provided scratch buffer.
//
// Limits: D <= kNoAllocMaxD (8192) and at most kNoAllocGroups (64) partial slots, i.e. 4 MiB of
// device memory that every GPU which loads this library holds until the process exits.
// The array is shared by all calls: two calls that overlap on the GPU (different streams) race on
// it.  Nothing in it has to start at zero - every slot that the reduction reads is rewritten by
// the first kernel of the same call - so the previous call's contents are harmless.
namespace {
constexpr int kNoAllocMaxD = 8192;
constexpr int kNoAllocGroups = 64;
static __device__ __align__(256) float g_norm_bwd_scratch[(size_t)kNoAllocGroups * 2 * kNoAllocMaxD];
// Device address of the array, resolved once per device.  In host code the symbol's name is only
// a stand-in; the kernels must be given the address that cudaGetSymbolAddress returns.
static float* g_norm_bwd_scratch_addr[64] = {nullptr};
}  // namespace

AX_API int ax_norm_bwd_noalloc(int rms, int act_dtype, int w_dtype, const void* dy, const void* x,
                               const void* w, const float* mean, const float* rstd,
                               const void* dres, void* dx, void* dw, void* db, int rows, int D,
                               cudaStream_t stream) {
  if (D % 8 != 0 || rows <= 0) return -1;
  if (D > kNoAllocMaxD) return -2;  // beyond the built-in scratch: use ax_norm_bwd with your own buffer
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -3;
  if (g_norm_bwd_scratch_addr[dev] == nullptr) {
    // First call on this device: resolve the array's device address (no allocation happens; the
    // array is part of the loaded module).  Do this before any stream capture.
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_norm_bwd_scratch);
    if (e != cudaSuccess) return (int)e;
    g_norm_bwd_scratch_addr[dev] = p;
  }
  int groups = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  if (groups > kNoAllocGroups) groups = kNoAllocGroups;
  return ax_norm_bwd(rms, act_dtype, w_dtype, dy, x, w, mean, rstd, dres, dx, dw, db,
                     g_norm_bwd_scratch_addr[dev], groups, rows, D, stream);
}

AX_API int ax_norm_bwd_noalloc_limits(int* max_d, int* max_groups) {
  *max_d = kNoAllocMaxD;
  *max_groups = kNoAllocGroups;
  return 0;
}
