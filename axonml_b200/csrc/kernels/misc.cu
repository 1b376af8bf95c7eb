// Embedding gather / scatter-add, rotary position embedding, dtype casts, strided copies.
//
// Parity: Embedding crates/axonml-nn/src/layers/embedding.rs:103 and the WGSL gather shader
// (wgpu_backend.rs:1527-1556); RoPE in the half-split convention of
// crates/axonml-llm/src/llama.rs:223-321; GPT-2 token+position embedding sum
// crates/axonml-llm/src/embedding.rs:335-365.
#include "common.cuh"

namespace {
using namespace ax;

template <typename T> __device__ __forceinline__ float ldv(const T* p) { return (float)*p; }
template <> __device__ __forceinline__ float ldv<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stv(T* p, float v) { *p = (T)v; }
template <> __device__ __forceinline__ void stv<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// out[t, :] = W[idx[t], :] (+ P[(t % S) + pos0, :])
template <typename T>
__global__ void embedding_fwd_kernel(const long* __restrict__ idx, const T* __restrict__ W,
                                     const T* __restrict__ P, T* __restrict__ out, long tokens,
                                     int D, int S, int pos0, long V, long padding_idx) {
  for (long t = blockIdx.x; t < tokens; t += gridDim.x) {
    long id = idx[t];
    const bool valid = id >= 0 && id < V;
    (void)AX_INB(id, 1, V, 2000);            // debug build: a token id outside the table is reported
    const T* w = W + (valid ? id : 0) * (long)D;
    const T* p = P ? P + ((long)(t % S) + pos0) * D : nullptr;
    T* o = out + t * D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float v = valid ? ldv(w + c) : 0.f;
      if (p) v += ldv(p + c);
      stv(o + c, v);
    }
  }
}

// dW[idx[t], :] += dout[t, :] (fp32 accumulation buffer); rows equal to padding_idx get nothing.
// dP[(t % S) + pos0, :] += dout[t, :] when dP is given.
template <typename T>
__global__ void embedding_bwd_kernel(const long* __restrict__ idx, const T* __restrict__ dout,
                                     float* __restrict__ dW, float* __restrict__ dP, long tokens,
                                     int D, int S, int pos0, long V, long padding_idx) {
  for (long t = blockIdx.x; t < tokens; t += gridDim.x) {
    long id = idx[t];
    (void)AX_INB(id, 1, V, 2001);
    const bool valid = id >= 0 && id < V && id != padding_idx;
    const T* g = dout + t * D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float v = ldv(g + c);
      if (valid) atomicAdd(dW + id * (long)D + c, v);
      if (dP) atomicAdd(dP + ((long)(t % S) + pos0) * D + c, v);
    }
  }
}

// In-place capable RoPE on x viewed as [tokens, heads, hd] with a token stride (elements).
// Token t has position pos0 + (t % S).  cos/sin tables are fp32 [max_pos, hd/2].
// sign = +1 forward, -1 backward (inverse rotation).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ cs,
                            const float* __restrict__ sn, long tokens, int heads, int hd,
                            long in_stride, long out_stride, int S, int pos0, float sign, int rot_heads,
                            const int* __restrict__ positions) {
  const int half = hd / 2;
  const long total = tokens * heads * half;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int j = (int)(i % half);
    const long th = i / half;
    const int hh = (int)(th % heads);
    const long t = th / heads;
    const long pos = positions ? (long)positions[t] : pos0 + (t % S);   // per-token positions (serving)
    const bool rot = hh < rot_heads;   // heads >= rot_heads are copied through unchanged
    const float c = rot ? cs[pos * half + j] : 1.f, s = rot ? sn[pos * half + j] * sign : 0.f;
    const T* xi = x + t * in_stride + (long)hh * hd;
    T* yo = y + t * out_stride + (long)hh * hd;
    const float a = ldv(xi + j), b = ldv(xi + j + half);
    stv(yo + j, a * c - b * s);
    stv(yo + j + half, b * c + a * s);
  }
}

template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ x, B* __restrict__ y, long n, float scale) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x)
    stv(y + i, ldv(x + i) * scale);
}

// 2-D tiled transpose: y[c, r] = x[r, c]
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols) {
  __shared__ T tile[32][33];
  int c = blockIdx.x * 32 + threadIdx.x, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y)
    if (r0 + j < rows && c < cols) tile[j][threadIdx.x] = x[(long)(r0 + j) * cols + c];
  __syncthreads();
  int r = r0 + threadIdx.x, c0 = blockIdx.x * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y)
    if (c0 + j < cols && r < rows) y[(long)(c0 + j) * rows + r] = tile[threadIdx.x][j];
}

inline int grid_for(long work, int block) {
  long g = (work + block - 1) / block;
  long cap = (long)axh::sm_count() * 16;
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

AX_API int ax_embedding_fwd(int dtype, const long* idx, const void* W, const void* P, void* out,
                            long tokens, int D, int S, int pos0, long V, long padding_idx,
                            cudaStream_t stream) {
  if (tokens <= 0) return 0;
  int grid = (int)(tokens < 65535 * 8 ? tokens : 65535 * 8);
  int block = D >= 1024 ? 256 : 128;
  if (dtype == 1)
    embedding_fwd_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
        idx, (const __nv_bfloat16*)W, (const __nv_bfloat16*)P, (__nv_bfloat16*)out, tokens, D,
        S < 1 ? 1 : S, pos0, V, padding_idx);
  else
    embedding_fwd_kernel<float><<<grid, block, 0, stream>>>(idx, (const float*)W, (const float*)P,
                                                            (float*)out, tokens, D, S < 1 ? 1 : S,
                                                            pos0, V, padding_idx);
  return (int)cudaGetLastError();
}

AX_API int ax_embedding_bwd(int dtype, const long* idx, const void* dout, float* dW, float* dP,
                            long tokens, int D, int S, int pos0, long V, long padding_idx,
                            cudaStream_t stream) {
  if (tokens <= 0) return 0;
  int grid = (int)(tokens < 65535 * 8 ? tokens : 65535 * 8);
  int block = D >= 1024 ? 256 : 128;
  if (dtype == 1)
    embedding_bwd_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
        idx, (const __nv_bfloat16*)dout, dW, dP, tokens, D, S < 1 ? 1 : S, pos0, V, padding_idx);
  else
    embedding_bwd_kernel<float><<<grid, block, 0, stream>>>(idx, (const float*)dout, dW, dP, tokens,
                                                            D, S < 1 ? 1 : S, pos0, V, padding_idx);
  return (int)cudaGetLastError();
}

AX_API int ax_rope(int dtype, const void* x, void* y, const float* cs, const float* sn, long tokens,
                   int heads, int hd, long in_stride, long out_stride, int S, int pos0, float sign,
                   int rot_heads, const int* positions, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hd % 2) return -1;
  long total = tokens * heads * (hd / 2);
  if (dtype == 1)
    rope_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)y, cs, sn, tokens, heads, hd, in_stride,
        out_stride, S < 1 ? 1 : S, pos0, sign, rot_heads, positions);
  else
    rope_kernel<float><<<grid_for(total, 256), 256, 0, stream>>>(
        (const float*)x, (float*)y, cs, sn, tokens, heads, hd, in_stride, out_stride,
        S < 1 ? 1 : S, pos0, sign, rot_heads, positions);
  return (int)cudaGetLastError();
}

// kinds: 0 = f32->bf16, 1 = bf16->f32, 2 = f32->f32 (scaled copy), 3 = bf16->bf16
AX_API int ax_cast(int kind, const void* x, void* y, long n, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  int g = grid_for(n, 256);
  switch (kind) {
    case 0: cast_kernel<float, __nv_bfloat16><<<g, 256, 0, stream>>>((const float*)x, (__nv_bfloat16*)y, n, scale); break;
    case 1: cast_kernel<__nv_bfloat16, float><<<g, 256, 0, stream>>>((const __nv_bfloat16*)x, (float*)y, n, scale); break;
    case 2: cast_kernel<float, float><<<g, 256, 0, stream>>>((const float*)x, (float*)y, n, scale); break;
    case 3: cast_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, scale); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

AX_API int ax_transpose(int dtype, const void* x, void* y, int rows, int cols,
                        cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  dim3 block(32, 8), grid((cols + 31) / 32, (rows + 31) / 32);
  if (dtype == 1)
    transpose_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, cols);
  else
    transpose_kernel<float><<<grid, block, 0, stream>>>((const float*)x, (float*)y, rows, cols);
  return (int)cudaGetLastError();
}
