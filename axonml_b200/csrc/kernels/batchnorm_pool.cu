// BatchNorm2d (training and inference) and MaxPool2d for NHWC bf16 activations.
//
// BatchNorm over [R = N*H*W rows, C channels], channels contiguous:
//   stats    : per-channel sum and sum of squares (fp32), one pass over x
//   finalize : mean, biased variance, rstd; scale = gamma*rstd, shift = beta - mean*scale; running
//              statistics running = (1-m)*running + m*batch with the BIASED variance, as the
//              reference does (crates/axonml-nn/src/layers/norm.rs:339-357)
//   apply    : y = relu?(x*scale + shift (+ residual)), one pass
//   backward : per-channel sums of dz and dz*xhat (dz = dy masked by y > 0 when ReLU was fused),
//              then dx = scale * (dz - mean(dz) - xhat * mean(dz*xhat)); dz is also the gradient
//              of the fused residual input
// Every pass moves 16 bytes per thread; partial sums are reduced in shared memory and added to the
// per-channel totals with one global reduction per CTA and channel.
//
// MaxPool2d (any window/stride/padding, NHWC): forward keeps the window position of the maximum
// (one byte per output element); backward gathers, for every input pixel, the output windows that
// selected it - no atomics.
//
// Replaces crates/axonml-nn/src/layers/norm.rs:285-378, pooling.rs:130-298 (CPU loops without
// gradients) and the WGSL shaders of wgpu_backend.rs:1430-1524.
#include "common.cuh"

namespace {
using namespace ax;

constexpr int kThreads = 256;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// Per-channel sums of f0(row) and f1(row) over the rows of this CTA's strip.
//   MODE 0: f0 = x, f1 = x*x
//   MODE 1: f0 = dz, f1 = dz * xhat, dz = dy (masked by y > 0 when `y` is given)
// Threads are laid out as (row lane, vector column): cv = C/8 vector columns, kThreads/cv row lanes.
template <int MODE>
__global__ void __launch_bounds__(kThreads)
bn_colsums_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ x,
                  const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean, const float* __restrict__ rstd,
                  float* __restrict__ sums, long R, int C) {
  extern __shared__ float red[];                 // [row lanes][2][C]
  const int cv = C / 8;
  const int lanes = kThreads / cv;
  const int vcol = threadIdx.x % cv, rl = threadIdx.x / cv;
  float s0[8], s1[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s0[j] = 0.f; s1[j] = 0.f; }
  float m[8], rs[8];
  if (MODE == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { m[j] = mean[vcol * 8 + j]; rs[j] = rstd[vcol * 8 + j]; }
  }
  if (rl < lanes) {
    for (long r = (long)blockIdx.x * lanes + rl; r < R; r += (long)gridDim.x * lanes) {
      float v[8];
      load8(a + r * C + vcol * 8, v);
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { s0[j] += v[j]; s1[j] += v[j] * v[j]; }
      } else {
        float xv[8];
        load8(x + r * C + vcol * 8, xv);
        if (y != nullptr) {
          float yv[8];
          load8(y + r * C + vcol * 8, yv);
#pragma unroll
          for (int j = 0; j < 8; ++j) if (!(yv[j] > 0.f)) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { s0[j] += v[j]; s1[j] += v[j] * (xv[j] - m[j]) * rs[j]; }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      red[(rl * 2 + 0) * C + vcol * 8 + j] = s0[j];
      red[(rl * 2 + 1) * C + vcol * 8 + j] = s1[j];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * C; i += kThreads) {
    float t = 0.f;
    for (int l = 0; l < lanes; ++l) t += red[l * 2 * C + i];
    atomicAdd(sums + i, t);
  }
}

__global__ void bn_finalize_kernel(const float* __restrict__ sums, const float* __restrict__ gamma,
                                   const float* __restrict__ beta, float* __restrict__ mean, float* __restrict__ rstd,
                                   float* __restrict__ scale, float* __restrict__ shift, float* __restrict__ run_mean,
                                   float* __restrict__ run_var, float momentum, float eps, float inv_rows, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float mu = sums[c] * inv_rows;
  const float var = fmaxf(sums[C + c] * inv_rows - mu * mu, 0.f);
  const float rs = rsqrtf(var + eps);
  mean[c] = mu;
  rstd[c] = rs;
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  scale[c] = g * rs;
  shift[c] = b - mu * g * rs;
  if (run_mean) {
    run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * mu;
    run_var[c] = (1.f - momentum) * run_var[c] + momentum * var;
  }
}

// inference: scale/shift from the running statistics
__global__ void bn_scale_shift_kernel(const float* __restrict__ gamma, const float* __restrict__ beta,
                                      const float* __restrict__ run_mean, const float* __restrict__ run_var,
                                      float* __restrict__ scale, float* __restrict__ shift, float eps, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float rs = rsqrtf(run_var[c] + eps);
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  scale[c] = g * rs;
  shift[c] = b - run_mean[c] * g * rs;
}

__global__ void __launch_bounds__(kThreads)
bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                const float* __restrict__ scale, const float* __restrict__ shift, __nv_bfloat16* __restrict__ y,
                long nvec, int C, int relu) {
  const int cv = C / 8;
  for (long i = (long)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += (long)gridDim.x * kThreads) {
    const int c0 = (int)(i % cv) * 8;
    float v[8];
    load8(x + i * 8, v);
    const float4 sa = *reinterpret_cast<const float4*>(scale + c0), sb = *reinterpret_cast<const float4*>(scale + c0 + 4);
    const float4 ha = *reinterpret_cast<const float4*>(shift + c0), hb = *reinterpret_cast<const float4*>(shift + c0 + 4);
    const float sc[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    const float sh[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = v[j] * sc[j] + sh[j];
    if (res != nullptr) {
      float r[8];
      load8(res + i * 8, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += r[j];
    }
    if (relu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
    }
    store8(y + i * 8, v);
  }
}

// dx = scale * (dz - s0/R - xhat * s1/R); dres = dz (when asked for)
__global__ void __launch_bounds__(kThreads)
bn_bwd_apply_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                    const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean, const float* __restrict__ rstd,
                    const float* __restrict__ scale, const float* __restrict__ sums, __nv_bfloat16* __restrict__ dx,
                    __nv_bfloat16* __restrict__ dres, long nvec, int C, float inv_rows) {
  const int cv = C / 8;
  for (long i = (long)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += (long)gridDim.x * kThreads) {
    const int c0 = (int)(i % cv) * 8;
    float g[8], xv[8];
    load8(dy + i * 8, g);
    load8(x + i * 8, xv);
    if (y != nullptr) {
      float yv[8];
      load8(y + i * 8, yv);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (!(yv[j] > 0.f)) g[j] = 0.f;
    }
    if (dres != nullptr) store8(dres + i * 8, g);
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j;
      const float xhat = (xv[j] - mean[c]) * rstd[c];
      o[j] = scale[c] * (g[j] - sums[c] * inv_rows - xhat * sums[C + c] * inv_rows);
    }
    store8(dx + i * 8, o);
  }
}

// ---------------------------------------------------------------------------- max pooling
// KT / ST: compile-time window and stride (0 = take the run-time values): with constants the window
// loops unroll and all loads of a window are in flight together.
template <int KT, int ST>
__global__ void __launch_bounds__(kThreads)
maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ idx,
                   int N, int H, int W, int C, int Ho, int Wo, int k_rt, int s_rt, int p) {
  const int k = KT ? KT : k_rt, s = ST ? ST : s_rt;
  const int cv = C / 8;
  const long total = (long)N * Ho * Wo * cv;
  for (long i = (long)blockIdx.x * kThreads + threadIdx.x; i < total; i += (long)gridDim.x * kThreads) {
    const int v = (int)(i % cv);
    long r = i / cv;
    const int wo = (int)(r % Wo); r /= Wo;
    const int ho = (int)(r % Ho);
    const int n = (int)(r / Ho);
    float best[8];
    int bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; bi[j] = 0; }
#pragma unroll
    for (int dh = 0; dh < k; ++dh) {
      const int h = ho * s - p + dh;
#pragma unroll
      for (int dw = 0; dw < k; ++dw) {
        const int w = wo * s - p + dw;
        if (h < 0 || h >= H || w < 0 || w >= W) continue;
        float t[8];
        load8(x + (((long)n * H + h) * W + w) * C + v * 8, t);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (t[j] > best[j]) { best[j] = t[j]; bi[j] = dh * k + dw; }
      }
    }
    store8(y + i * 8, best);
    if (idx != nullptr) {
      uint2 pk;
      pk.x = bi[0] | (bi[1] << 8) | (bi[2] << 16) | (bi[3] << 24);
      pk.y = bi[4] | (bi[5] << 8) | (bi[6] << 16) | (bi[7] << 24);
      *reinterpret_cast<uint2*>(idx + i * 8) = pk;
    }
  }
}

template <int KT, int ST>
__global__ void __launch_bounds__(kThreads)
maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const uint8_t* __restrict__ idx, __nv_bfloat16* __restrict__ dx,
                   int N, int H, int W, int C, int Ho, int Wo, int k_rt, int s_rt, int p) {
  const int k = KT ? KT : k_rt, s = ST ? ST : s_rt;
  // a pixel lies in at most ceil(k/s) windows per axis
  constexpr int kMaxWin = (KT && ST) ? (KT + ST - 1) / ST : 0;
  const int cv = C / 8;
  const long total = (long)N * H * W * cv;
  for (long i = (long)blockIdx.x * kThreads + threadIdx.x; i < total; i += (long)gridDim.x * kThreads) {
    const int v = (int)(i % cv);
    long r = i / cv;
    const int w = (int)(r % W); r /= W;
    const int h = (int)(r % H);
    const int n = (int)(r / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // output windows that contain (h, w): ho*s - p <= h < ho*s - p + k
    const int ho_lo = max(0, (h + p - k + s) / s), ho_hi = min(Ho - 1, (h + p) / s);
    const int wo_lo = max(0, (w + p - k + s) / s), wo_hi = min(Wo - 1, (w + p) / s);
#pragma unroll
    for (int a = 0; a < (kMaxWin ? kMaxWin : 1 << 30); ++a) {
      const int ho = ho_lo + a;
      if (ho > ho_hi) break;
      const int dh = h - (ho * s - p);
      if (dh < 0 || dh >= k) continue;
#pragma unroll
      for (int b = 0; b < (kMaxWin ? kMaxWin : 1 << 30); ++b) {
        const int wo = wo_lo + b;
        if (wo > wo_hi) break;
        const int dw = w - (wo * s - p);
        if (dw < 0 || dw >= k) continue;
        const long o = ((((long)n * Ho + ho) * Wo + wo) * cv + v) * 8;
        const uint2 pk = *reinterpret_cast<const uint2*>(idx + o);
        float g[8];
        load8(dy + o, g);
        const int want = dh * k + dw;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int sel = ((j < 4 ? pk.x : pk.y) >> (8 * (j & 3))) & 0xff;
          if (sel == want) acc[j] += g[j];
        }
      }
    }
    store8(dx + i * 8, acc);
  }
}

int grid_for(long work_items) {
  long g = (work_items + kThreads - 1) / kThreads;
  const long cap = (long)axh::sm_count() * 8;
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

// Training forward.  x, res (optional), y: [R, C] bf16; gamma/beta/run_mean/run_var: fp32 [C] (optional);
// mean/rstd/scale/shift: fp32 [C] outputs (saved for backward); sums: fp32 [2*C] scratch, zero on entry.
// C must be a multiple of 8 and at most 2048.
AX_API int ax_batchnorm_fwd_train(const void* x, const void* res, const float* gamma, const float* beta, void* y,
                                  float* mean, float* rstd, float* scale, float* shift, float* run_mean,
                                  float* run_var, float* sums, long R, int C, float momentum, float eps, int relu,
                                  cudaStream_t stream) {
  if (R <= 0) return 0;
  if (C % 8 || C > 2048 || C < 8) return -1;
  const int cv = C / 8;
  const int lanes = kThreads / cv;
  if (lanes < 1) return -1;
  long strips = (R + lanes - 1) / lanes;
  int grid = (int)(strips < (long)axh::sm_count() * 4 ? strips : (long)axh::sm_count() * 4);
  const size_t smem = (size_t)lanes * 2 * C * sizeof(float);
  bn_colsums_kernel<0><<<grid, kThreads, smem, stream>>>((const __nv_bfloat16*)x, nullptr, nullptr, nullptr, nullptr,
                                                         sums, R, C);
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, stream>>>(sums, gamma, beta, mean, rstd, scale, shift, run_mean, run_var,
                                                          momentum, eps, 1.0f / (float)R, C);
  const long nvec = R * cv;
  bn_apply_kernel<<<grid_for(nvec), kThreads, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, scale, shift,
                                                           (__nv_bfloat16*)y, nvec, C, relu);
  return (int)cudaGetLastError();
}

// Inference forward with the running statistics.  scale/shift: fp32 [C] scratch.
AX_API int ax_batchnorm_fwd_eval(const void* x, const void* res, const float* gamma, const float* beta,
                                 const float* run_mean, const float* run_var, void* y, float* scale, float* shift,
                                 long R, int C, float eps, int relu, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (C % 8) return -1;
  bn_scale_shift_kernel<<<(C + 127) / 128, 128, 0, stream>>>(gamma, beta, run_mean, run_var, scale, shift, eps, C);
  const long nvec = R * (C / 8);
  bn_apply_kernel<<<grid_for(nvec), kThreads, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, scale, shift,
                                                           (__nv_bfloat16*)y, nvec, C, relu);
  return (int)cudaGetLastError();
}

// Backward of the training forward.  y: the forward output when ReLU was fused, else null.
// sums: fp32 [2*C], zero on entry; on return sums[0:C] = dbeta, sums[C:2C] = dgamma.
// dres (optional) receives the gradient of the fused residual input.
AX_API int ax_batchnorm_bwd(const void* dy, const void* x, const void* y, const float* mean, const float* rstd,
                            const float* scale, void* dx, void* dres, float* sums, long R, int C,
                            cudaStream_t stream) {
  if (R <= 0) return 0;
  if (C % 8 || C > 2048 || C < 8) return -1;
  const int cv = C / 8;
  const int lanes = kThreads / cv;
  long strips = (R + lanes - 1) / lanes;
  int grid = (int)(strips < (long)axh::sm_count() * 4 ? strips : (long)axh::sm_count() * 4);
  const size_t smem = (size_t)lanes * 2 * C * sizeof(float);
  bn_colsums_kernel<1><<<grid, kThreads, smem, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                         (const __nv_bfloat16*)y, mean, rstd, sums, R, C);
  const long nvec = R * cv;
  bn_bwd_apply_kernel<<<grid_for(nvec), kThreads, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                               (const __nv_bfloat16*)y, mean, rstd, scale, sums,
                                                               (__nv_bfloat16*)dx, (__nv_bfloat16*)dres, nvec, C,
                                                               1.0f / (float)R);
  return (int)cudaGetLastError();
}

// x [N, H, W, C] -> y [N, Ho, Wo, C] bf16; idx (optional, one byte per output element) records the
// window position of the maximum for the backward pass.  C multiple of 8, k*k <= 255.
AX_API int ax_maxpool2d_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, int k, int s, int p,
                            cudaStream_t stream) {
  if (C % 8 || k < 1 || k * k > 255 || s < 1) return -1;
  const int Ho = (H + 2 * p - k) / s + 1, Wo = (W + 2 * p - k) / s + 1;
  if (N <= 0 || Ho <= 0 || Wo <= 0) return 0;
  const long total = (long)N * Ho * Wo * (C / 8);
  if (k == 3 && s == 2)
    maxpool_fwd_kernel<3, 2><<<grid_for(total), kThreads, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y,
                                                                       (uint8_t*)idx, N, H, W, C, Ho, Wo, k, s, p);
  else if (k == 2 && s == 2)
    maxpool_fwd_kernel<2, 2><<<grid_for(total), kThreads, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y,
                                                                       (uint8_t*)idx, N, H, W, C, Ho, Wo, k, s, p);
  else
    maxpool_fwd_kernel<0, 0><<<grid_for(total), kThreads, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y,
                                                                       (uint8_t*)idx, N, H, W, C, Ho, Wo, k, s, p);
  return (int)cudaGetLastError();
}

AX_API int ax_maxpool2d_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int k, int s, int p,
                            cudaStream_t stream) {
  if (C % 8 || k < 1 || k * k > 255 || s < 1) return -1;
  const int Ho = (H + 2 * p - k) / s + 1, Wo = (W + 2 * p - k) / s + 1;
  if (N <= 0 || Ho <= 0 || Wo <= 0) return 0;
  const long total = (long)N * H * W * (C / 8);
  if (k == 3 && s == 2)
    maxpool_bwd_kernel<3, 2><<<grid_for(total), kThreads, 0, stream>>>((const __nv_bfloat16*)dy, (const uint8_t*)idx,
                                                                       (__nv_bfloat16*)dx, N, H, W, C, Ho, Wo, k, s, p);
  else if (k == 2 && s == 2)
    maxpool_bwd_kernel<2, 2><<<grid_for(total), kThreads, 0, stream>>>((const __nv_bfloat16*)dy, (const uint8_t*)idx,
                                                                       (__nv_bfloat16*)dx, N, H, W, C, Ho, Wo, k, s, p);
  else
    maxpool_bwd_kernel<0, 0><<<grid_for(total), kThreads, 0, stream>>>((const __nv_bfloat16*)dy, (const uint8_t*)idx,
                                                                       (__nv_bfloat16*)dx, N, H, W, C, Ho, Wo, k, s, p);
  return (int)cudaGetLastError();
}
