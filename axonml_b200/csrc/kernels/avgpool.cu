// Average pooling, forward and backward, for 4-D activations in either memory layout (NCHW or
// channels-last), fp32 or bf16, fp32 accumulation.  One kernel covers the three layers of the
// reference (crates/axonml-nn/src/layers/pooling.rs:120-200 AvgPool1d as H = 1, :296-357 AvgPool2d,
// :384-445 AdaptiveAvgPool2d) through its window rule:
//
//   fixed    window of output (oh, ow) = rows [oh*sh - ph, oh*sh - ph + kh) x cols likewise, clipped to
//            the image; the divisor is the number of pixels inside the image (the reference's rule),
//            or kh*kw when `count_pad` is set (the torch default);
//   adaptive rows [floor(oh*H/OH), floor((oh+1)*H/OH)) (the reference's rule: the windows partition
//            the image; an empty window gives 0).
//
// The forward runs one thread per output element, the backward one thread per input element that
// adds up the outputs whose window contains it (no atomics, deterministic).  Threads are numbered
// along the contiguous dimension of the layout, so loads and stores coalesce in both layouts.
#include "common.cuh"

namespace {
using namespace ax;

struct PoolParams {
  int N, C, H, W, OH, OW;
  int kh, kw, sh, sw, ph, pw;
  int adaptive, count_pad, channels_last;
};

__device__ __forceinline__ void window(const PoolParams& p, int o, int size, int osize, int k, int s, int pad,
                                       int& lo, int& hi, int& span) {
  if (p.adaptive) {
    lo = (int)(((long)o * size) / osize);
    hi = (int)(((long)(o + 1) * size) / osize);
    span = hi - lo;
  } else {
    lo = o * s - pad;
    hi = lo + k;
    span = k;
    if (lo < 0) lo = 0;
    if (hi > size) hi = size;
  }
}

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void from_f(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// linear thread id -> (n, c, a, b) with the layout's contiguous dimension fastest
__device__ __forceinline__ void decode(long i, int C, int A, int B, int channels_last, int& n, int& c, int& a, int& b) {
  if (channels_last) {
    c = (int)(i % C); i /= C;
    b = (int)(i % B); i /= B;
    a = (int)(i % A); n = (int)(i / A);
  } else {
    b = (int)(i % B); i /= B;
    a = (int)(i % A); i /= A;
    c = (int)(i % C); n = (int)(i / C);
  }
}
__device__ __forceinline__ long offset(int n, int c, int a, int b, int C, int A, int B, int channels_last) {
  return channels_last ? (((long)n * A + a) * B + b) * C + c : (((long)n * C + c) * A + a) * B + b;
}

template <typename T>
__global__ void __launch_bounds__(256) avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, const PoolParams p) {
  const long total = (long)p.N * p.C * p.OH * p.OW;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int n, c, oh, ow;
    decode(i, p.C, p.OH, p.OW, p.channels_last, n, c, oh, ow);
    int h0, h1, hs, w0, w1, ws;
    window(p, oh, p.H, p.OH, p.kh, p.sh, p.ph, h0, h1, hs);
    window(p, ow, p.W, p.OW, p.kw, p.sw, p.pw, w0, w1, ws);
    float acc = 0.f;
    const long in_total = (long)p.N * p.C * p.H * p.W;
    for (int h = h0; h < h1; ++h)
      for (int w = w0; w < w1; ++w) {
        const long off = offset(n, c, h, w, p.C, p.H, p.W, p.channels_last);
        if (AX_INB(off, 1, in_total, 3000)) acc += to_f(x[off]);
      }
    const int cnt = (!p.adaptive && p.count_pad) ? hs * ws : max(h1 - h0, 0) * max(w1 - w0, 0);
    from_f(&y[i], cnt > 0 ? acc / (float)cnt : 0.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, const PoolParams p) {
  const long total = (long)p.N * p.C * p.H * p.W;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int n, c, h, w;
    decode(i, p.C, p.H, p.W, p.channels_last, n, c, h, w);
    // candidate outputs: every window that can contain (h, w)
    int oh_lo, oh_hi, ow_lo, ow_hi;
    if (p.adaptive) {
      // windows are [floor(o*H/OH), floor((o+1)*H/OH)): o is at most floor(((h+1)*OH - 1)/H) and at least that minus one step
      oh_hi = min(p.OH - 1, (int)((((long)h + 1) * p.OH - 1) / p.H));
      oh_lo = max(0, (int)(((long)h * p.OH) / p.H) - 1);
      ow_hi = min(p.OW - 1, (int)((((long)w + 1) * p.OW - 1) / p.W));
      ow_lo = max(0, (int)(((long)w * p.OW) / p.W) - 1);
    } else {
      oh_lo = max(0, (h + p.ph - p.kh + p.sh) / p.sh);       // ceil((h + ph - kh + 1) / sh) for the non-negative case
      if (h + p.ph - p.kh + 1 <= 0) oh_lo = 0;
      oh_hi = min(p.OH - 1, (h + p.ph) / p.sh);
      ow_lo = max(0, (w + p.pw - p.kw + p.sw) / p.sw);
      if (w + p.pw - p.kw + 1 <= 0) ow_lo = 0;
      ow_hi = min(p.OW - 1, (w + p.pw) / p.sw);
    }
    float acc = 0.f;
    for (int oh = oh_lo; oh <= oh_hi; ++oh) {
      int h0, h1, hs;
      window(p, oh, p.H, p.OH, p.kh, p.sh, p.ph, h0, h1, hs);
      if (h < h0 || h >= h1) continue;
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        int w0, w1, ws;
        window(p, ow, p.W, p.OW, p.kw, p.sw, p.pw, w0, w1, ws);
        if (w < w0 || w >= w1) continue;
        const int cnt = (!p.adaptive && p.count_pad) ? hs * ws : (h1 - h0) * (w1 - w0);
        const long off = offset(n, c, oh, ow, p.C, p.OH, p.OW, p.channels_last);
        if (AX_INB(off, 1, (long)p.N * p.C * p.OH * p.OW, 3001)) acc += to_f(dy[off]) / (float)cnt;
      }
    }
    from_f(&dx[i], acc);
  }
}

int launch(int bwd, int bf16, const void* in, void* out, const PoolParams& p, cudaStream_t stream) {
  const long total = (long)p.N * p.C * (bwd ? (long)p.H * p.W : (long)p.OH * p.OW);
  if (total <= 0) return 0;
  long blocks = (total + 255) / 256;
  const long cap = (long)axh::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (bwd) {
    if (bf16) avgpool_bwd_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, p);
    else avgpool_bwd_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)in, (float*)out, p);
  } else {
    if (bf16) avgpool_fwd_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, p);
    else avgpool_fwd_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)in, (float*)out, p);
  }
  return (int)cudaGetLastError();
}

}  // namespace

// dims: int[6] = N, C, H, W, OH, OW;  win: int[6] = kh, kw, sh, sw, ph, pw (ignored when adaptive);
// dtype: 0 fp32, 1 bf16.  Forward: in = x [N,C,H,W], out = y [N,C,OH,OW]; backward: in = dy, out = dx.
// Both tensors use the layout named by `channels_last` and are dense in it.
AX_API int ax_avgpool2d(int backward, int dtype, const void* in, void* out, const int* dims, const int* win,
                        int adaptive, int count_pad, int channels_last, cudaStream_t stream) {
  PoolParams p;
  p.N = dims[0]; p.C = dims[1]; p.H = dims[2]; p.W = dims[3]; p.OH = dims[4]; p.OW = dims[5];
  p.kh = win[0]; p.kw = win[1]; p.sh = win[2]; p.sw = win[3]; p.ph = win[4]; p.pw = win[5];
  p.adaptive = adaptive; p.count_pad = count_pad; p.channels_last = channels_last;
  if (p.N < 0 || p.C <= 0 || p.H <= 0 || p.W <= 0 || p.OH <= 0 || p.OW <= 0) return -1;
  if (!adaptive && (p.kh <= 0 || p.kw <= 0 || p.sh <= 0 || p.sw <= 0 || p.ph < 0 || p.pw < 0)) return -1;
  return launch(backward, dtype, in, out, p, stream);
}
