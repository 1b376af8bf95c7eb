// Block quantisation on the GPU: quantise fp32/bf16 -> Q8_0 / Q4_0 / Q4_1 / Q5_0 / Q5_1 / Q4_K and dequantise every GGML block
// format this package reads (Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q4_K) to bf16 or fp32.  Layouts are the
// GGML ones, identical to the CPU codecs in csrc/host/quant.cpp, so tensors quantised here can be
// written to a GGUF file unchanged.
//
// Parity: crates/axonml-quant/src/quantize.rs:82-205 and dequantize.rs:20-125 (rayon CPU loops).
#include "common.cuh"

namespace {
using namespace ax;

template <typename T> __device__ __forceinline__ float ldx(const T* p, long i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, long i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stx(T* p, long i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, long i, float v) { p[i] = __float2bfloat16(v); }

__device__ __forceinline__ float h2f(const uint8_t* p) {
  return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}
__device__ __forceinline__ void f2h(uint8_t* p, float v) {
  // every block starts on an even byte, so the scale is one aligned 16-bit store
  *reinterpret_cast<__half*>(p) = __float2half_rn(v);
}
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& d, int& m) {
  if (j < 4) { d = q[j] & 63; m = q[j + 4] & 63; }
  else { d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// one warp per 32-element block
template <typename T>
__global__ void quantize_q8_0_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, long nblocks) {
  const long b = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  const float v = ldx(x, b * 32 + lane);
  const float amax = warp_max(fabsf(v));
  const float d = amax / 127.f, id = d > 0.f ? 1.f / d : 0.f;
  uint8_t* o = out + b * 34;
  if (lane == 0) f2h(o, d);
  int q = __float2int_rn(v * id);
  q = max(-127, min(127, q));
  o[2 + lane] = (uint8_t)(int8_t)q;
}

// Q4_0 / Q4_1 / Q5_0 / Q5_1: one warp per 32-element block, lane l owns element l.  The rules are
// those of the CPU codec (scale = absmax / 7 or 15 for the symmetric formats, (max - min) / 15 or 31
// with a stored minimum for the others; round to nearest even; GGML nibble order: elements j and
// j + 16 share a byte, the fifth bits go to a 32-bit mask).
template <typename T, int TYPE>
__global__ void quantize_q45_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, long nblocks) {
  constexpr bool kFive = TYPE == 3 || TYPE == 4;
  constexpr bool kMin = TYPE == 2 || TYPE == 4;
  constexpr int kBytes = TYPE == 1 ? 18 : TYPE == 2 ? 20 : TYPE == 3 ? 22 : 24;
  constexpr int kHdr = kMin ? 4 : 2;
  constexpr int kTop = kFive ? 31 : 15;
  const long b = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  const float v = ldx(x, b * 32 + lane);
  float mn = v, mx = v;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const float amax = fmaxf(fabsf(mn), fabsf(mx));
  // correctly rounded division and reciprocal (the library is built with fast-math, whose
  // approximate division would move a value that sits on a rounding boundary)
  const float d = kMin ? __fdiv_rn(mx - mn, (float)kTop) : __fdiv_rn(amax, (float)(kTop / 2));
  const float id = d != 0.f ? __frcp_rn(d) : 0.f;
  int q;
  if (kMin) q = max(0, min(kTop, __float2int_rn(__fmul_rn(__fsub_rn(v, mn), id))));
  else q = max(-(kTop + 1) / 2, min(kTop / 2, __float2int_rn(__fmul_rn(v, id)))) + (kTop + 1) / 2;
  uint8_t* o = out + b * kBytes;
  if (lane == 0) {
    f2h(o, d);
    if (kMin) f2h(o + 2, mn);
  }
  const int hi_q = __shfl_down_sync(0xffffffffu, q, 16);       // element lane + 16, for lanes 0..15
  if (lane < 16) o[kHdr + (kFive ? 4 : 0) + lane] = (uint8_t)((q & 0xF) | ((hi_q & 0xF) << 4));
  if (kFive) {
    const uint32_t qh = __ballot_sync(0xffffffffu, (q >> 4) & 1);   // bit l = fifth bit of element l
    if (lane == 0) {
      o[kHdr + 0] = (uint8_t)(qh & 0xFF); o[kHdr + 1] = (uint8_t)((qh >> 8) & 0xFF);
      o[kHdr + 2] = (uint8_t)((qh >> 16) & 0xFF); o[kHdr + 3] = (uint8_t)(qh >> 24);
    }
  }
}

// one warp per 256-element super-block; lane l owns elements [8l, 8l+8) (sub-block l/4)
template <typename T>
__global__ void quantize_q4_k_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, long nblocks) {
  const long b = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  float v[8];
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = ldx(x, b * 256 + lane * 8 + i);
    mn = fminf(mn, v[i]);
    mx = fmaxf(mx, v[i]);
  }
  // min / max over the 4 lanes of a sub-block
  mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 1)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 2)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  if (mn > 0.f) mn = 0.f;
  const float scale = (mx > mn) ? (mx - mn) / 15.f : 0.f;
  const float minv = -mn;
  // super-block maxima over the 8 sub-blocks
  float ms = scale, mm = minv;
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    ms = fmaxf(ms, __shfl_xor_sync(0xffffffffu, ms, o));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
  }
  const float inv_s = ms > 0.f ? 63.f / ms : 0.f, inv_m = mm > 0.f ? 63.f / mm : 0.f;
  const int ls = min(63, __float2int_rn(inv_s * scale)), lm = min(63, __float2int_rn(inv_m * minv));
  const float dd = __half2float(__float2half_rn(ms / 63.f)), dm = __half2float(__float2half_rn(mm / 63.f));
  uint8_t* o = out + b * 144;
  // gather the 8 (ls, lm) pairs on every lane
  int lsj[8], lmj[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { lsj[j] = __shfl_sync(0xffffffffu, ls, j * 4); lmj[j] = __shfl_sync(0xffffffffu, lm, j * 4); }
  if (lane == 0) {
    f2h(o, ms / 63.f);
    f2h(o + 2, mm / 63.f);
    uint8_t sc[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) sc[i] = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < 4) { sc[j] = (uint8_t)lsj[j]; sc[j + 4] = (uint8_t)lmj[j]; }
      else {
        sc[j + 4] = (uint8_t)((lsj[j] & 0xF) | ((lmj[j] & 0xF) << 4));
        sc[j - 4] |= (uint8_t)((lsj[j] >> 4) << 6);
        sc[j] |= (uint8_t)((lmj[j] >> 4) << 6);
      }
    }
#pragma unroll
    for (int i = 0; i < 12; ++i) o[4 + i] = sc[i];
  }
  const float d = dd * ls, m = dm * lm;
  const float id = d > 0.f ? 1.f / d : 0.f;
  uint32_t nib = 0;   // my 8 codes, 4 bits each
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int q = __float2int_rn((v[i] + m) * id);
    q = max(0, min(15, q));
    nib |= (uint32_t)q << (4 * i);
  }
  // 64-element chunk c = lane/8; lanes with (lane%8) < 4 hold the low-nibble half, their partner
  // lane+4 the high-nibble half of the same 32 bytes
  const uint32_t other = __shfl_down_sync(0xffffffffu, nib, 4);
  if ((lane & 7) < 4) {
    uint8_t* q = o + 16 + (lane >> 3) * 32 + (lane & 7) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = (uint8_t)(((nib >> (4 * i)) & 0xF) | (((other >> (4 * i)) & 0xF) << 4));
  }
}

// generic dequantise: one thread per block of 32 elements (Q4_K: per 32-element sub-block)
template <typename T>
__global__ void dequantize_kernel(int type, const uint8_t* __restrict__ in, T* __restrict__ y, long nsub) {
  const long s = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= nsub) return;
  T* o = y + s * 32;
  if (type == 0) {
    const uint8_t* b = in + s * 34;
    const float d = h2f(b);
    for (int i = 0; i < 32; ++i) stx(o, i, d * (float)(int8_t)b[2 + i]);
  } else if (type == 1 || type == 2) {
    const uint8_t* b = in + s * (type == 1 ? 18 : 20);
    const float d = h2f(b), m = type == 2 ? h2f(b + 2) : 0.f;
    const uint8_t* q = b + (type == 1 ? 2 : 4);
    for (int i = 0; i < 16; ++i) {
      const int lo = q[i] & 0xF, hi = q[i] >> 4;
      stx(o, i, type == 1 ? d * (lo - 8) : d * lo + m);
      stx(o, i + 16, type == 1 ? d * (hi - 8) : d * hi + m);
    }
  } else if (type == 3 || type == 4) {
    const uint8_t* b = in + s * (type == 3 ? 22 : 24);
    const int hdr = type == 3 ? 2 : 4;
    const float d = h2f(b), m = type == 4 ? h2f(b + 2) : 0.f;
    const uint32_t qh = b[hdr] | (b[hdr + 1] << 8) | (b[hdr + 2] << 16) | ((uint32_t)b[hdr + 3] << 24);
    const uint8_t* q = b + hdr + 4;
    for (int i = 0; i < 16; ++i) {
      const int lo = (q[i] & 0xF) | (((qh >> i) & 1) << 4), hi = (q[i] >> 4) | (((qh >> (i + 16)) & 1) << 4);
      stx(o, i, type == 3 ? d * (lo - 16) : d * lo + m);
      stx(o, i + 16, type == 3 ? d * (hi - 16) : d * hi + m);
    }
  } else {
    const long sb = s >> 3;
    const int j = (int)(s & 7);
    const uint8_t* b = in + sb * 144;
    const float d = h2f(b), dmin = h2f(b + 2);
    int sc, mn;
    scale_min_k4(j, b + 4, sc, mn);
    const float dl = d * sc, ml = dmin * mn;
    const uint8_t* q = b + 16 + (j >> 1) * 32;
    for (int i = 0; i < 32; ++i) stx(o, i, dl * ((j & 1) ? (q[i] >> 4) : (q[i] & 0xF)) - ml);
  }
}

}  // namespace

// type ids as in csrc/host/quant.cpp: 0 Q8_0, 1 Q4_0, 2 Q4_1, 3 Q5_0, 4 Q5_1, 5 Q4_K
AX_API int ax_quantize_cuda(int type, int in_bf16, const void* x, void* out, long n, cudaStream_t stream) {
  if (type == 0) {
    if (n % 32) return -1;
    const long nb = n / 32;
    const int grid = (int)((nb * 32 + 255) / 256);
    if (in_bf16) quantize_q8_0_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (uint8_t*)out, nb);
    else quantize_q8_0_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (uint8_t*)out, nb);
  } else if (type == 5) {
    if (n % 256) return -1;
    const long nb = n / 256;
    const int grid = (int)((nb * 32 + 255) / 256);
    if (in_bf16) quantize_q4_k_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (uint8_t*)out, nb);
    else quantize_q4_k_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (uint8_t*)out, nb);
  } else if (type >= 1 && type <= 4) {
    if (n % 32) return -1;
    const long nb = n / 32;
    const int grid = (int)((nb * 32 + 255) / 256);
#define AX_Q45(TY)                                                                                         \
    if (type == TY) {                                                                                      \
      if (in_bf16) quantize_q45_kernel<__nv_bfloat16, TY><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (uint8_t*)out, nb); \
      else quantize_q45_kernel<float, TY><<<grid, 256, 0, stream>>>((const float*)x, (uint8_t*)out, nb);   \
    }
    AX_Q45(1) AX_Q45(2) AX_Q45(3) AX_Q45(4)
#undef AX_Q45
  } else {
    return -2;
  }
  return (int)cudaGetLastError();
}

AX_API int ax_dequantize_cuda(int type, int out_bf16, const void* in, void* y, long n, cudaStream_t stream) {
  if (type < 0 || type > 5 || n % (type == 5 ? 256 : 32)) return -1;
  const long nsub = n / 32;
  const int grid = (int)((nsub + 127) / 128);
  if (out_bf16) dequantize_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(type, (const uint8_t*)in, (__nv_bfloat16*)y, nsub);
  else dequantize_kernel<float><<<grid, 128, 0, stream>>>(type, (const uint8_t*)in, (float*)y, nsub);
  return (int)cudaGetLastError();
}
