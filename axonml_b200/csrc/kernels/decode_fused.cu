// Producers of int8 activations for the decode matrix-vector kernels, and the RoPE + KV-cache write
// of a decode step in one launch.
//
// The matrix-vector kernels (qgemv.cu) multiply packed weights with activations quantised to int8 in
// blocks of 32 (scale dx and scaled block sum sx per block, as llama.cpp's Q8_1).  A decode step at
// batch 1 is a chain of launches of a few microseconds each, so every launch that only reshapes
// data costs as much as a real one.  Here the operations that PRODUCE the input of a matrix-vector
// product write it in that int8 form directly:
//
//   rmsnorm_q8      x (+ residual) -> updated residual stream (bf16) and q8(rmsnorm(x) * w)
//   swiglu_q8       gate|up        -> q8(silu(gate) * up)
//   rope_kv_write   packed q|k|v   -> rotated q (contiguous), rotated k and v into the paged cache
//   q8_rows         plain quantiser (inputs that come from another library kernel)
//
// The merge kernel of the paged attention (paged_attn.cu) has the same int8 epilogue.
//
// The reference's decode path runs dequantise -> fp32 matmul per layer on the CPU
// (crates/axonml-quant/src/dequantize.rs:20-125, crates/axonml-llm/src/attention.rs:19-86).
#include "common.cuh"

namespace {
using namespace ax;

// Quantises the 32 values held by the 4 lanes of a quad (8 each, consecutive) and stores them.
// `mask`: the lanes of the warp that make this call (whole quads).
__device__ __forceinline__ void q8_store_quad(unsigned mask, const float (&v)[8], int8_t* x8, float* dx, float* sx,
                                              long elem0, long blk, int quad_lane) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
  const float d = amax / 127.f;
  const float id = d > 0.f ? 1.f / d : 0.f;
  int q[8], s = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) { q[i] = __float2int_rn(v[i] * id); s += q[i]; }
  s += __shfl_xor_sync(mask, s, 1);
  s += __shfl_xor_sync(mask, s, 2);
  uint2 o;
  o.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
  o.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
  *reinterpret_cast<uint2*>(x8 + elem0) = o;
  if (quad_lane == 0) { dx[blk] = d; sx[blk] = d * (float)s; }
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = e.x; v[7] = e.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]); u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

constexpr int kNormThreads = 256;
constexpr int kNormChunks = 8;       // 8-element chunks per thread: rows of up to 16384 values

// One CTA per row.  Thread t holds chunks t, t + 256, ...; the four lanes of a quad hold one
// 32-value quantisation block.
template <typename WT>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_q8_kernel(const __nv_bfloat16* __restrict__ x, long ldx, const __nv_bfloat16* __restrict__ add, long ldadd,
                  const WT* __restrict__ w, float eps, __nv_bfloat16* __restrict__ x_out, long ldout,
                  __nv_bfloat16* __restrict__ h_out, long ldh, int8_t* __restrict__ x8, float* __restrict__ dx,
                  float* __restrict__ sx, int K) {
  __shared__ float red[kNormThreads / 32];
  const int row = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nchunks = K / 8;
  float v[kNormChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int ch = t + c * kNormThreads;
    if (ch < nchunks) {
      load8(x + (long)row * ldx + ch * 8, v[c]);
      if (add != nullptr) {
        float a[8];
        load8(add + (long)row * ldadd + ch * 8, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += a[i];
        // the residual stream continues in bf16: normalise what the next layer will read
        if (x_out != nullptr) store8(x_out + (long)row * ldout + ch * 8, v[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] = __bfloat162float(__float2bfloat16(v[c][i]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[c][i] * v[c][i];
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)K + eps);
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int ch = t + c * kNormThreads;
    const unsigned mask = __ballot_sync(0xffffffffu, ch < nchunks);
    if (ch < nchunks) {                       // whole quads are in or out: K is a multiple of 32
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wi = sizeof(WT) == 2 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[ch * 8 + i])
                                         : reinterpret_cast<const float*>(w)[ch * 8 + i];
        // the bf16 rounding of the unfused path (norm output stored as bf16, then quantised)
        y[i] = __bfloat162float(__float2bfloat16(v[c][i] * rstd * wi));
      }
      if (h_out != nullptr) store8(h_out + (long)row * ldh + ch * 8, y);
      q8_store_quad(mask, y, x8 + (long)row * K, dx + (long)row * (K / 32), sx + (long)row * (K / 32), (long)ch * 8, ch >> 2,
                    lane & 3);
    }
  }
}

// One quad per 32-value block of the product; gate|up halves of a row of 2F values.
__global__ void __launch_bounds__(256)
swiglu_q8_kernel(const __nv_bfloat16* __restrict__ gu, long ld, int8_t* __restrict__ x8, float* __restrict__ dx,
                 float* __restrict__ sx, int B, int F) {
  const long chunk = (long)blockIdx.x * blockDim.x + threadIdx.x;      // 8 values each
  const int per_row = F / 8;
  const unsigned mask = __ballot_sync(0xffffffffu, chunk < (long)B * per_row);
  if (chunk >= (long)B * per_row) return;                               // F % 32 == 0: quads are never split
  const int b = (int)(chunk / per_row), ch = (int)(chunk - (long)b * per_row);
  float g[8], u[8], y[8];
  load8(gu + (long)b * ld + ch * 8, g);
  load8(gu + (long)b * ld + F + ch * 8, u);
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = __bfloat162float(__float2bfloat16(g[i] / (1.f + __expf(-g[i])) * u[i]));
  q8_store_quad(mask, y, x8 + (long)b * F, dx + (long)b * (F / 32), sx + (long)b * (F / 32), (long)ch * 8, ch >> 2,
                threadIdx.x & 3);
}

__global__ void __launch_bounds__(256)
q8_rows_kernel(const __nv_bfloat16* __restrict__ x, long ld, int8_t* __restrict__ x8, float* __restrict__ dx,
               float* __restrict__ sx, int B, int K) {
  const long chunk = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = K / 8;
  const unsigned mask = __ballot_sync(0xffffffffu, chunk < (long)B * per_row);
  if (chunk >= (long)B * per_row) return;
  const int b = (int)(chunk / per_row), ch = (int)(chunk - (long)b * per_row);
  float y[8];
  load8(x + (long)b * ld + ch * 8, y);
  q8_store_quad(mask, y, x8 + (long)b * K, dx + (long)b * (K / 32), sx + (long)b * (K / 32), (long)ch * 8, ch >> 2,
                threadIdx.x & 3);
}

// Grid (B, Hq + 2 Hkv): one CTA of 64 threads per head of a token; thread j owns the pair
// (j, j + 64) of the 128-wide head (half-split rotation).
__global__ void __launch_bounds__(64)
rope_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, long ld, const float* __restrict__ cs,
                     const float* __restrict__ sn, const int* __restrict__ positions, __nv_bfloat16* __restrict__ q_out,
                     __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table,
                     const int* __restrict__ seq_ids, int Hq, int Hkv, int page_size, int max_pages) {
  constexpr int D = 128, half = 64;
  const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int pos = positions[b];
  const __nv_bfloat16* src = qkv + (long)b * ld + (long)h * D;
  float a = __bfloat162float(src[j]), c = __bfloat162float(src[j + half]);
  if (h < Hq + Hkv) {
    const float co = cs[(long)pos * half + j], si = sn[(long)pos * half + j];
    const float ra = a * co - c * si, rc = c * co + a * si;
    a = ra; c = rc;
  }
  __nv_bfloat16* dst;
  if (h < Hq) {
    dst = q_out + ((long)b * Hq + h) * D;
  } else {
    const int page = block_table[(long)seq_ids[b] * max_pages + pos / page_size];
    const long row = ((long)page * page_size + pos % page_size) * ((long)Hkv * D);
    dst = (h < Hq + Hkv) ? kc + row + (long)(h - Hq) * D : vc + row + (long)(h - Hq - Hkv) * D;
  }
  dst[j] = __float2bfloat16(a);
  dst[j + half] = __float2bfloat16(c);
}

}  // namespace

// q8(x[B, K]) with K % 32 == 0; x rows 16-byte aligned (ld % 8 == 0).
AX_API int ax_q8_rows(const void* x, long ld, void* x8, float* dx, float* sx, int B, int K, cudaStream_t stream) {
  if (B <= 0 || K <= 0) return 0;
  if (K % 32 || ld % 8 || (((uintptr_t)x | (uintptr_t)x8) & 15)) return -1;
  const long chunks = (long)B * (K / 8);
  q8_rows_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x, ld, (int8_t*)x8, dx, sx, B, K);
  return (int)cudaGetLastError();
}

// xs = x + add (when add is given; stored to x_out when that is given), y = rmsnorm(xs) * w,
// quantised into x8 / dx / sx and optionally stored as bf16 in h_out.  K % 32 == 0, K <= 16384.
// w_kind: 1 fp32, 2 bf16.
AX_API int ax_rmsnorm_q8(const void* x, long ldx, const void* add, long ldadd, const void* w, int w_kind, float eps,
                         void* x_out, long ldout, void* h_out, long ldh, void* x8, float* dx, float* sx, int B, int K,
                         cudaStream_t stream) {
  if (B <= 0) return 0;
  if (K <= 0 || K % 32 || K > kNormThreads * kNormChunks * 8) return -1;
  if ((ldx | ldadd | ldout | ldh) % 8) return -1;
  if (((uintptr_t)x | (uintptr_t)add | (uintptr_t)x_out | (uintptr_t)h_out | (uintptr_t)x8) & 15) return -1;
  if (w_kind == 1)
    rmsnorm_q8_kernel<float><<<B, kNormThreads, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)add, ldadd,
                                                             (const float*)w, eps, (__nv_bfloat16*)x_out, ldout,
                                                             (__nv_bfloat16*)h_out, ldh, (int8_t*)x8, dx, sx, K);
  else if (w_kind == 2)
    rmsnorm_q8_kernel<__nv_bfloat16><<<B, kNormThreads, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)add,
                                                                     ldadd, (const __nv_bfloat16*)w, eps,
                                                                     (__nv_bfloat16*)x_out, ldout, (__nv_bfloat16*)h_out, ldh,
                                                                     (int8_t*)x8, dx, sx, K);
  else
    return -1;
  return (int)cudaGetLastError();
}

// q8(silu(gate) * up) of gu[B, 2F] (gate | up); F % 32 == 0.
AX_API int ax_swiglu_q8(const void* gu, long ld, void* x8, float* dx, float* sx, int B, int F, cudaStream_t stream) {
  if (B <= 0 || F <= 0) return 0;
  if (F % 32 || ld % 8 || (((uintptr_t)gu | (uintptr_t)x8) & 15)) return -1;
  const long chunks = (long)B * (F / 8);
  swiglu_q8_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, ld, (int8_t*)x8, dx, sx, B, F);
  return (int)cudaGetLastError();
}

// Decode step: qkv [B, Hq + 2 Hkv, 128] bf16 (row stride ld) -> q_out [B, Hq, 128] rotated, and the
// rotated key and the value of each token into the pages of its sequence at its position.
AX_API int ax_rope_kv_write(const void* qkv, long ld, const float* cs, const float* sn, const int* positions,
                            void* q_out, void* kc, void* vc, const int* block_table, const int* seq_ids, int B, int Hq,
                            int Hkv, int Dh, int page_size, int max_pages, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Dh != 128 || page_size <= 0 || Hq + 2 * Hkv > 65535) return -1;
  rope_kv_write_kernel<<<dim3(B, Hq + 2 * Hkv), 64, 0, stream>>>((const __nv_bfloat16*)qkv, ld, cs, sn, positions,
                                                                 (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc,
                                                                 (__nv_bfloat16*)vc, block_table, seq_ids, Hq, Hkv,
                                                                 page_size, max_pages);
  return (int)cudaGetLastError();
}
