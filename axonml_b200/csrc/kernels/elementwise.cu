// Elementwise / activation kernel set: vectorised (16-byte) grid-stride kernels, one
// instantiation per opcode (a switch per element costs more instructions than the memory system
// leaves room for at HBM speed).  Covers the reference's CUDA island (cuda_kernels/elementwise.cu, activations.cu:
// add, sub, mul, div, scale, add_scalar, neg, abs, sqrt, pow, pow_scalar, clamp, relu, sigmoid,
// tanh, leaky_relu, exp, log, gelu, silu, elu and the three *_backward kernels) and the
// arithmetic of its WGSL/MSL compute shaders (wgpu_backend.rs:1003-1267, metal.rs:527-700),
// plus SwiGLU, activation backward for the fused Linear epilogues, and Philox dropout.
#include "common.cuh"

namespace {
using namespace ax;

enum UnaryOp : int {
  U_NEG = 0, U_ABS, U_SQRT, U_EXP, U_LOG, U_RELU, U_SIGMOID, U_TANH, U_GELU, U_SILU, U_ELU,
  U_LEAKY_RELU, U_SCALE, U_ADD_SCALAR, U_POW_SCALAR, U_CLAMP, U_SQUARE, U_RSQRT, U_COPY,
};
enum BinaryOp : int {
  B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_MAX, B_MIN,
  // backward forms: out = f(dy=a, saved=b)
  B_RELU_BWD, B_SIGMOID_BWD, B_TANH_BWD, B_GELU_BWD, B_SILU_BWD, B_ELU_BWD, B_LEAKY_RELU_BWD,
  // out = a + alpha*b
  B_AXPY,
};

__device__ __forceinline__ float unary(float x, int op, float p0, float p1) {
  switch (op) {
    case U_NEG: return -x;
    case U_ABS: return fabsf(x);
    case U_SQRT: return sqrtf(x);
    case U_EXP: return __expf(x);
    case U_LOG: return __logf(x);
    case U_RELU: return fmaxf(x, 0.f);
    case U_SIGMOID: return sigmoidf_(x);
    case U_TANH: return tanhf(x);
    case U_GELU: return gelu_tanh(x);
    case U_SILU: return siluf_(x);
    case U_ELU: return x > 0.f ? x : p0 * (__expf(x) - 1.f);
    case U_LEAKY_RELU: return x > 0.f ? x : p0 * x;
    case U_SCALE: return x * p0;
    case U_ADD_SCALAR: return x + p0;
    case U_POW_SCALAR: return powf(x, p0);
    case U_CLAMP: return fminf(fmaxf(x, p0), p1);
    case U_SQUARE: return x * x;
    case U_RSQRT: return rsqrtf(x);
    default: return x;
  }
}

__device__ __forceinline__ float binary(float a, float b, int op, float p0) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return a / b;
    case B_POW: return powf(a, b);
    case B_MAX: return fmaxf(a, b);
    case B_MIN: return fminf(a, b);
    case B_RELU_BWD: return b > 0.f ? a : 0.f;                    // b = input x
    case B_SIGMOID_BWD: return a * b * (1.f - b);                 // b = output s
    case B_TANH_BWD: return a * (1.f - b * b);                    // b = output t
    case B_GELU_BWD: return a * gelu_tanh_grad(b);                // b = input x
    case B_SILU_BWD: { float s = sigmoidf_(b); return a * (s + b * s * (1.f - s)); }
    case B_ELU_BWD: return b > 0.f ? a : a * p0 * __expf(b);      // b = input x
    case B_LEAKY_RELU_BWD: return b > 0.f ? a : a * p0;
    case B_AXPY: return a + p0 * b;
    default: return a;
  }
}

template <typename T> struct IO;
template <> struct IO<float> {
  static constexpr int V = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  static __device__ __forceinline__ float ld1(const float* p) { return *p; }
  static __device__ __forceinline__ void st1(float* p, float v) { *p = v; }
};
template <> struct IO<__nv_bfloat16> {
  static constexpr int V = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
    u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st1(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

template <typename T, int op>
__global__ void unary_kernel(const T* __restrict__ x, T* __restrict__ y, long n, float p0,
                             float p1, int aligned) {
  constexpr int V = IO<T>::V;
  const long stride = (long)gridDim.x * blockDim.x;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long nv = aligned ? n / V : 0;
  for (long i = tid; i < nv; i += stride) {
    if (!AX_INB(i * V, V, n, 1000)) continue;
    float v[V];
    IO<T>::load(x + i * V, v);
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = unary(v[j], op, p0, p1);
    IO<T>::store(y + i * V, v);
  }
  for (long i = nv * V + tid; i < n; i += stride) {
    if (!AX_INB(i, 1, n, 1001)) continue;
    IO<T>::st1(y + i, unary(IO<T>::ld1(x + i), op, p0, p1));
  }
}

template <typename T, int op>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y,
                              long n, float p0, int aligned) {
  constexpr int V = IO<T>::V;
  const long stride = (long)gridDim.x * blockDim.x;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long nv = aligned ? n / V : 0;
  for (long i = tid; i < nv; i += stride) {
    float va[V], vb[V];
    IO<T>::load(a + i * V, va);
    IO<T>::load(b + i * V, vb);
#pragma unroll
    for (int j = 0; j < V; ++j) va[j] = binary(va[j], vb[j], op, p0);
    IO<T>::store(y + i * V, va);
  }
  for (long i = nv * V + tid; i < n; i += stride)
    IO<T>::st1(y + i, binary(IO<T>::ld1(a + i), IO<T>::ld1(b + i), op, p0));
}

// SwiGLU on a fused [rows, 2*H] gate|up tensor: out[r, h] = silu(gu[r, h]) * gu[r, H + h]
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, long rows, int H) {
  constexpr int V = IO<T>::V;
  const long per_row = H / V;
  const long total = rows * per_row;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const long r = i / per_row;
    const int c = (int)(i - r * per_row) * V;
    float g[V], u[V];
    IO<T>::load(gu + r * 2 * H + c, g);
    IO<T>::load(gu + r * 2 * H + H + c, u);
#pragma unroll
    for (int j = 0; j < V; ++j) g[j] = siluf_(g[j]) * u[j];
    IO<T>::store(out + r * H + c, g);
  }
}

// d(gate|up)[r, :] from dout[r, :]
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ gu,
                                  T* __restrict__ dgu, long rows, int H) {
  constexpr int V = IO<T>::V;
  const long per_row = H / V;
  const long total = rows * per_row;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const long r = i / per_row;
    const int c = (int)(i - r * per_row) * V;
    float g[V], u[V], d[V], dg[V], du[V];
    IO<T>::load(gu + r * 2 * H + c, g);
    IO<T>::load(gu + r * 2 * H + H + c, u);
    IO<T>::load(dout + r * H + c, d);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float s = sigmoidf_(g[j]);
      dg[j] = d[j] * u[j] * (s + g[j] * s * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    IO<T>::store(dgu + r * 2 * H + c, dg);
    IO<T>::store(dgu + r * 2 * H + H + c, du);
  }
}

// Philox-4x32-10 counter RNG
__device__ __forceinline__ uint4 philox(uint64_t seed, uint64_t ctr) {
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0, c3 = 0;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// y = x * mask / (1-p); mask (uint8) is written for the backward pass.
template <typename T>
__global__ void dropout_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                   uint8_t* __restrict__ mask, long n, float p, uint64_t seed,
                                   uint64_t offset) {
  const float scale = 1.f / (1.f - p);
  const long groups = (n + 3) / 4;
  for (long g = (long)blockIdx.x * blockDim.x + threadIdx.x; g < groups;
       g += (long)gridDim.x * blockDim.x) {
    uint4 r = philox(seed, offset + (uint64_t)g);
    uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      long i = g * 4 + j;
      if (i < n) {
        bool keep = (rr[j] * 2.3283064365386963e-10f) >= p;
        if (mask) mask[i] = keep ? 1 : 0;
        IO<T>::st1(y + i, keep ? IO<T>::ld1(x + i) * scale : 0.f);
      }
    }
  }
}

template <typename T>
__global__ void dropout_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ mask,
                                   T* __restrict__ dx, long n, float p) {
  const float scale = 1.f / (1.f - p);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x)
    IO<T>::st1(dx + i, mask[i] ? IO<T>::ld1(dy + i) * scale : 0.f);
}

// column sums of a [rows, N] matrix (bias gradient): out[n] = sum_r x[r, n], fp32 out.
// grid.x covers N in chunks of 32 columns x 8 (vector); rows are split over blockDim.y.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ x, float* __restrict__ out, long rows, int N,
                              long ld) {
  __shared__ float sm[32][33];
  const int col = blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (col < N)
    for (long r = (long)blockIdx.y * blockDim.y + threadIdx.y; r < rows; r += (long)gridDim.y * blockDim.y)
      acc += IO<T>::ld1(x + r * ld + col);
  sm[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < N) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) t += sm[j][threadIdx.x];
    atomicAdd(out + col, t);
  }
}

// Vectorised column sums: a thread owns V adjacent columns (one 16-byte load per row), a warp 32*V
// adjacent columns, the 8 warps of a block (and gridDim.y blocks) split the rows.
template <typename T>
__global__ void __launch_bounds__(256) colsum_vec_kernel(const T* __restrict__ x, float* __restrict__ out, long rows,
                                                        int N, long ld) {
  constexpr int V = IO<T>::V;
  __shared__ float sm[8][32 * V + 1];
  const int col = (blockIdx.x * 32 + threadIdx.x) * V;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  if (col < N) {
    long r = (long)blockIdx.y * 8 + threadIdx.y;
    const long step = (long)gridDim.y * 8;
    // two rows in flight per thread
    for (; r + step < rows; r += 2 * step) {
      float a[V], b[V];
      IO<T>::load(x + r * ld + col, a);
      IO<T>::load(x + (r + step) * ld + col, b);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += a[j] + b[j];
    }
    for (; r < rows; r += step) {
      float a[V];
      IO<T>::load(x + r * ld + col, a);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += a[j];
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) sm[threadIdx.y][threadIdx.x * V + j] = acc[j];
  __syncthreads();
  for (int c = threadIdx.y * 32 + threadIdx.x; c < 32 * V; c += 256) {
    const int gc = blockIdx.x * 32 * V + c;
    if (gc < N) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sm[w][c];
      atomicAdd(out + gc, t);
    }
  }
}

inline int grid_for(long work, int block) {
  long g = (work + block - 1) / block;
  long cap = (long)axh::sm_count() * 16;
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

inline bool aligned16(const void* a, const void* b, const void* c) {
  return ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c)) & 15) == 0;
}

}  // namespace

template <int OP>
static void launch_unary(int dtype, const void* x, void* y, long n, float p0, float p1, int al, cudaStream_t stream) {
  if (dtype == 1)
    unary_kernel<__nv_bfloat16, OP><<<grid_for(n / 8 + 1, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y,
                                                                                  n, p0, p1, al);
  else
    unary_kernel<float, OP><<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>((const float*)x, (float*)y, n, p0, p1, al);
}

AX_API int ax_unary(int dtype, int op, const void* x, void* y, long n, float p0, float p1,
                    cudaStream_t stream) {
  if (n <= 0) return 0;
  const int al = aligned16(x, y, nullptr);
#define AX_U(OP) case OP: launch_unary<OP>(dtype, x, y, n, p0, p1, al, stream); break;
  switch (op) {
    AX_U(U_NEG) AX_U(U_ABS) AX_U(U_SQRT) AX_U(U_EXP) AX_U(U_LOG) AX_U(U_RELU) AX_U(U_SIGMOID) AX_U(U_TANH)
    AX_U(U_GELU) AX_U(U_SILU) AX_U(U_ELU) AX_U(U_LEAKY_RELU) AX_U(U_SCALE) AX_U(U_ADD_SCALAR) AX_U(U_POW_SCALAR)
    AX_U(U_CLAMP) AX_U(U_SQUARE) AX_U(U_RSQRT) AX_U(U_COPY)
    default: return -1;
  }
#undef AX_U
  return (int)cudaGetLastError();
}

template <int OP>
static void launch_binary(int dtype, const void* a, const void* b, void* y, long n, float p0, int al, cudaStream_t stream) {
  if (dtype == 1)
    binary_kernel<__nv_bfloat16, OP><<<grid_for(n / 8 + 1, 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n, p0, al);
  else
    binary_kernel<float, OP><<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>((const float*)a, (const float*)b, (float*)y, n,
                                                                           p0, al);
}

AX_API int ax_binary(int dtype, int op, const void* a, const void* b, void* y, long n, float p0,
                     cudaStream_t stream) {
  if (n <= 0) return 0;
  const int al = aligned16(a, b, y);
#define AX_B(OP) case OP: launch_binary<OP>(dtype, a, b, y, n, p0, al, stream); break;
  switch (op) {
    AX_B(B_ADD) AX_B(B_SUB) AX_B(B_MUL) AX_B(B_DIV) AX_B(B_POW) AX_B(B_MAX) AX_B(B_MIN) AX_B(B_RELU_BWD)
    AX_B(B_SIGMOID_BWD) AX_B(B_TANH_BWD) AX_B(B_GELU_BWD) AX_B(B_SILU_BWD) AX_B(B_ELU_BWD) AX_B(B_LEAKY_RELU_BWD)
    AX_B(B_AXPY)
    default: return -1;
  }
#undef AX_B
  return (int)cudaGetLastError();
}

AX_API int ax_swiglu_fwd(int dtype, const void* gu, void* out, long rows, int H,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1) {
    if (H % 8) return -1;
    swiglu_fwd_kernel<__nv_bfloat16><<<grid_for(rows * (H / 8), 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, H);
  } else {
    if (H % 4) return -1;
    swiglu_fwd_kernel<float><<<grid_for(rows * (H / 4), 256), 256, 0, stream>>>(
        (const float*)gu, (float*)out, rows, H);
  }
  return (int)cudaGetLastError();
}

AX_API int ax_swiglu_bwd(int dtype, const void* dout, const void* gu, void* dgu, long rows, int H,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1) {
    if (H % 8) return -1;
    swiglu_bwd_kernel<__nv_bfloat16><<<grid_for(rows * (H / 8), 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, rows, H);
  } else {
    if (H % 4) return -1;
    swiglu_bwd_kernel<float><<<grid_for(rows * (H / 4), 256), 256, 0, stream>>>(
        (const float*)dout, (const float*)gu, (float*)dgu, rows, H);
  }
  return (int)cudaGetLastError();
}

AX_API int ax_dropout_fwd(int dtype, const void* x, void* y, uint8_t* mask, long n, float p,
                          uint64_t seed, uint64_t offset, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == 1)
    dropout_fwd_kernel<__nv_bfloat16><<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)y, mask, n, p, seed, offset);
  else
    dropout_fwd_kernel<float><<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>(
        (const float*)x, (float*)y, mask, n, p, seed, offset);
  return (int)cudaGetLastError();
}

AX_API int ax_dropout_bwd(int dtype, const void* dy, const uint8_t* mask, void* dx, long n, float p,
                          cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == 1)
    dropout_bwd_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)dy, mask, (__nv_bfloat16*)dx, n, p);
  else
    dropout_bwd_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)dy, mask,
                                                                    (float*)dx, n, p);
  return (int)cudaGetLastError();
}

// out (fp32, [N]) must be zeroed by the caller.
AX_API int ax_colsum(int dtype, const void* x, float* out, long rows, int N, long ld,
                     cudaStream_t stream) {
  if (rows <= 0 || N <= 0) return 0;
  const int V = dtype == 1 ? 8 : 4;
  if (N % V == 0 && ld % V == 0 && (((uintptr_t)x) & 15) == 0) {
    dim3 block(32, 8);
    const int gx = (N + 32 * V - 1) / (32 * V);
    long gy = (long)axh::sm_count() * 8 / gx;            // about eight blocks per SM
    if (gy > (rows + 15) / 16) gy = (rows + 15) / 16;
    if (gy < 1) gy = 1;
    dim3 grid(gx, (unsigned)gy);
    if (dtype == 1)
      colsum_vec_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)x, out, rows, N, ld);
    else
      colsum_vec_kernel<float><<<grid, block, 0, stream>>>((const float*)x, out, rows, N, ld);
    return (int)cudaGetLastError();
  }
  dim3 block(32, 32);
  int gy = (int)((rows + 1023) / 1024);
  if (gy > 64) gy = 64;
  if (gy < 1) gy = 1;
  dim3 grid((N + 31) / 32, gy);
  if (dtype == 1)
    colsum_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)x, out, rows, N, ld);
  else
    colsum_kernel<float><<<grid, block, 0, stream>>>((const float*)x, out, rows, N, ld);
  return (int)cudaGetLastError();
}
