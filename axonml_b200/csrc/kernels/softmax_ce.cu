// Row softmax / log-softmax (forward and backward) and the fused cross-entropy
// (log-softmax + NLL) forward and backward.  One CTA per row, online max/sum in fp32,
// 16-byte vector loads when the row is aligned.
//
// Cross-entropy keeps only the per-row log-sum-exp between forward and backward; backward
// recomputes the probabilities from the logits, so no [rows, V] probability tensor is stored.
// `row_stride` may exceed `V` (vocabularies padded for the GEMM that produced the logits).
//
// Parity: crates/axonml-nn/src/loss.rs:166-204 (CrossEntropyLoss), functional.rs:85 (softmax),
// cuda_kernels/activations.cu:162-185 (softmax_f32, one thread per row in the reference).
#include "common.cuh"

namespace {
using namespace ax;

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long i) {
  return __bfloat162float(p[i]);
}
template <typename T>
__device__ __forceinline__ void stf(T* p, long i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long i, float v) {
  p[i] = __float2bfloat16(v);
}

constexpr int kThreads = 512;

// one 16-byte chunk of a row as floats
__device__ __forceinline__ void load_chunk(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void load_chunk(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void store_chunk(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_chunk(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ void online_combine(float& m, float& s, float m2, float s2) {
  float mn = fmaxf(m, m2);
  if (mn == -INFINITY) { m = mn; s = 0.f; return; }
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

// block-wide (max, sum-exp) of a row
template <typename T>
__device__ __forceinline__ void row_max_sum(const T* row, int V, float& m_out, float& s_out) {
  __shared__ float sm[kThreads / 32], ss[kThreads / 32];
  float m = -INFINITY, s = 0.f;
  // 16-byte chunks first (8 bf16 / 4 fp32): one running-max update per chunk instead of a
  // data-dependent branch per element
  constexpr int kVec = 16 / (int)sizeof(T);
  const int nvec = (((uintptr_t)row & 15) == 0) ? V / kVec : 0;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float v[kVec];
    load_chunk(row + (long)i * kVec, v);
    float mx = v[0];
#pragma unroll
    for (int j = 1; j < kVec; ++j) mx = fmaxf(mx, v[j]);
    if (mx > m) { s *= __expf(m - mx); m = mx; }
    if (m != -INFINITY) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) s += __expf(v[j] - m);
    }
  }
  for (int i = nvec * kVec + threadIdx.x; i < V; i += blockDim.x) {
    float v = ldf(row, i);
    if (v > m) { s = s * __expf(m - v) + 1.f; m = v; }
    else s += __expf(v - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_combine(m, s, m2, s2);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    m = lane < nw ? sm[lane] : -INFINITY;
    s = lane < nw ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_combine(m, s, m2, s2);
    }
    if (lane == 0) { sm[0] = m; ss[0] = s; }
  }
  __syncthreads();
  m_out = sm[0];
  s_out = ss[0];
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int V, long stride, int log_mode) {
  const T* row = x + (long)blockIdx.x * stride;
  T* out = y + (long)blockIdx.x * stride;
  float m, s;
  row_max_sum(row, V, m, s);
  const float lse = m + __logf(s);
  const float inv = 1.f / s;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = ldf(row, i);
    stf(out, i, log_mode ? v - lse : __expf(v - m) * inv);
  }
}

// softmax:     dx = y * (dy - sum(dy*y));  log-softmax: dx = dy - exp(y) * sum(dy)
template <typename T>
__global__ void __launch_bounds__(kThreads)
softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int V,
                   long stride, int log_mode) {
  __shared__ float red[kThreads / 32];
  const T* dyr = dy + (long)blockIdx.x * stride;
  const T* yr = y + (long)blockIdx.x * stride;
  T* dxr = dx + (long)blockIdx.x * stride;
  float acc = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float g = ldf(dyr, i);
    acc += log_mode ? g : g * ldf(yr, i);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float g = ldf(dyr, i), yy = ldf(yr, i);
    stf(dxr, i, log_mode ? g - __expf(yy) * tot : yy * (g - tot));
  }
}

// loss[row] = lse - logit[target]; rows whose target == ignore_index give 0.
template <typename T>
__global__ void __launch_bounds__(kThreads)
ce_fwd_kernel(const T* __restrict__ logits, const long* __restrict__ target,
              float* __restrict__ loss, float* __restrict__ lse_out, int V, long stride,
              long ignore_index) {
  const T* row = logits + (long)blockIdx.x * stride;
  float m, s;
  row_max_sum(row, V, m, s);
  if (threadIdx.x == 0) {
    const float lse = m + __logf(s);
    lse_out[blockIdx.x] = lse;
    const long t = target[blockIdx.x];
    (void)AX_INB(t == ignore_index ? 0 : t, 1, V, 5000);     // debug build: a class index outside the vocabulary is reported
    loss[blockIdx.x] = (t == ignore_index || t < 0 || t >= V) ? 0.f : lse - ldf(row, t);
  }
}

// stats[row] = {row max, sum exp(x - max), x[target] if 0 <= target < V else 0, unused}
template <typename T>
__global__ void __launch_bounds__(kThreads)
vp_ce_stats_kernel(const T* __restrict__ logits, const long* __restrict__ target, float* __restrict__ stats,
                   int V, long stride) {
  const T* row = logits + (long)blockIdx.x * stride;
  float m = -INFINITY, s = 0.f;
  if (V > 0) row_max_sum(row, V, m, s);
  if (threadIdx.x == 0) {
    const long t = target[blockIdx.x];
    float4 o;
    o.x = m; o.y = s; o.z = (t >= 0 && t < V) ? ldf(row, t) : 0.f; o.w = 0.f;
    *reinterpret_cast<float4*>(stats + (long)blockIdx.x * 4) = o;
  }
}

// dlogits = (softmax - onehot) * gscale[row or 0]; columns in [V, stride_cols) are zeroed so
// that a padded vocabulary contributes nothing to the following GEMMs.
template <typename T>
__global__ void __launch_bounds__(kThreads)
ce_bwd_kernel(const T* __restrict__ logits, const long* __restrict__ target,
              const float* __restrict__ lse, const float* __restrict__ gscale, int gscale_per_row,
              float gmul, T* __restrict__ dlogits, int V, int Vpad, long stride,
              long ignore_index, int partial) {
  const T* row = logits + (long)blockIdx.x * stride;
  T* out = dlogits + (long)blockIdx.x * stride;
  const long t = target[blockIdx.x];
  // `partial`: the row is one rank's slice of a vocabulary split over ranks and `lse` is the
  // log-sum-exp over the whole vocabulary; a target outside [0, V) then lives on another rank, so
  // the row still gets its softmax share and only the one-hot term is missing
  const bool ignored = partial ? (t == ignore_index) : (t == ignore_index || t < 0 || t >= V);
  const float g = ignored ? 0.f : gmul * (gscale ? gscale[gscale_per_row ? blockIdx.x : 0] : 1.f);
  const float l = lse[blockIdx.x];
  constexpr int kVec = 16 / (int)sizeof(T);
  const bool vec_ok = ((((uintptr_t)row) | ((uintptr_t)out)) & 15) == 0;
  const int nvec = vec_ok ? V / kVec : 0;          // chunks that lie entirely inside the vocabulary
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float v[kVec];
    if (ignored) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) v[j] = 0.f;
    } else {
      load_chunk(row + (long)i * kVec, v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) v[j] = __expf(v[j] - l) * g;
      const long rel = t - (long)i * kVec;
      if (rel >= 0 && rel < kVec) {
#pragma unroll
        for (int j = 0; j < kVec; ++j)
          if (j == (int)rel) v[j] -= g;
      }
    }
    store_chunk(out + (long)i * kVec, v);
  }
  for (int i = nvec * kVec + threadIdx.x; i < Vpad; i += blockDim.x) {
    float v = 0.f;
    if (i < V && !ignored) {
      v = __expf(ldf(row, i) - l);
      if (i == t) v -= 1.f;
      v *= g;
    }
    stf(out, i, v);
  }
}

// sum of a float vector scaled (used for the mean/sum loss reduction) - single CTA
__global__ void reduce_sum_kernel(const float* __restrict__ x, float* __restrict__ out, long n,
                                  float scale) {
  __shared__ float red[32];
  float acc = 0.f;
  for (long i = threadIdx.x; i < n; i += blockDim.x) acc += x[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) out[0] = v * scale;
  }
}

// number of targets != ignore_index (as float) - single CTA
__global__ void count_valid_kernel(const long* __restrict__ target, float* __restrict__ out,
                                   long n, long ignore_index, int V) {
  __shared__ float red[32];
  float acc = 0.f;
  for (long i = threadIdx.x; i < n; i += blockDim.x) {
    long t = target[i];
    acc += (t == ignore_index || t < 0 || t >= V) ? 0.f : 1.f;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) out[0] = v;
  }
}

}  // namespace

AX_API int ax_softmax_fwd(int dtype, const void* x, void* y, int rows, int V, long stride,
                          int log_mode, cudaStream_t stream) {
  if (rows <= 0 || V <= 0) return 0;
  if (dtype == 1)
    softmax_fwd_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)y, V, stride, log_mode);
  else
    softmax_fwd_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)x, (float*)y, V, stride,
                                                             log_mode);
  return (int)cudaGetLastError();
}

AX_API int ax_softmax_bwd(int dtype, const void* dy, const void* y, void* dx, int rows, int V,
                          long stride, int log_mode, cudaStream_t stream) {
  if (rows <= 0 || V <= 0) return 0;
  if (dtype == 1)
    softmax_bwd_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, (__nv_bfloat16*)dx, V, stride, log_mode);
  else
    softmax_bwd_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)dy, (const float*)y,
                                                             (float*)dx, V, stride, log_mode);
  return (int)cudaGetLastError();
}

AX_API int ax_ce_fwd(int dtype, const void* logits, const long* target, float* loss, float* lse,
                     int rows, int V, long stride, long ignore_index, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1)
    ce_fwd_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)logits,
                                                                 target, loss, lse, V, stride,
                                                                 ignore_index);
  else
    ce_fwd_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, target, loss, lse, V,
                                                        stride, ignore_index);
  return (int)cudaGetLastError();
}

AX_API int ax_ce_bwd(int dtype, const void* logits, const long* target, const float* lse,
                     const float* gscale, int gscale_per_row, float gmul, void* dlogits, int rows,
                     int V, int Vpad, long stride, long ignore_index, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1)
    ce_bwd_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>(
        (const __nv_bfloat16*)logits, target, lse, gscale, gscale_per_row, gmul,
        (__nv_bfloat16*)dlogits, V, Vpad, stride, ignore_index, 0);
  else
    ce_bwd_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, target, lse, gscale,
                                                        gscale_per_row, gmul, (float*)dlogits, V,
                                                        Vpad, stride, ignore_index, 0);
  return (int)cudaGetLastError();
}

// Vocabulary-parallel cross-entropy, this rank's part (the class dimension of the logits is split
// over the ranks of a tensor-parallel group):
//  stats: per row {max, sum exp(x - max), logit of the target or 0} over this rank's V columns; the
//         target index is relative to this rank's first column, outside [0, V) = not on this rank.
//         The caller combines the rows' statistics over the ranks (one small collective).
//  bwd:   dlogits = (exp(x - lse) - onehot) * scale with the log-sum-exp over the WHOLE vocabulary
//         and the one-hot term only where the target is on this rank.
AX_API int ax_vp_ce_stats(int dtype, const void* logits, const long* local_target, float* stats, int rows, int V,
                          long stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1)
    vp_ce_stats_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)logits, local_target, stats, V, stride);
  else
    vp_ce_stats_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, local_target, stats, V, stride);
  return (int)cudaGetLastError();
}

AX_API int ax_vp_ce_bwd(int dtype, const void* logits, const long* local_target, const float* lse,
                        const float* gscale, float gmul, void* dlogits, int rows, int V, int Vpad, long stride,
                        long ignore_index, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1)
    ce_bwd_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)logits, local_target, lse, gscale, 0, gmul,
                                                                 (__nv_bfloat16*)dlogits, V, Vpad, stride, ignore_index, 1);
  else
    ce_bwd_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, local_target, lse, gscale, 0, gmul,
                                                        (float*)dlogits, V, Vpad, stride, ignore_index, 1);
  return (int)cudaGetLastError();
}

AX_API int ax_reduce_sum_f32(const float* x, float* out, long n, float scale,
                             cudaStream_t stream) {
  reduce_sum_kernel<<<1, 1024, 0, stream>>>(x, out, n, scale);
  return (int)cudaGetLastError();
}

AX_API int ax_count_valid(const long* target, float* out, long n, long ignore_index, int V,
                          cudaStream_t stream) {
  count_valid_kernel<<<1, 1024, 0, stream>>>(target, out, n, ignore_index, V);
  return (int)cudaGetLastError();
}
