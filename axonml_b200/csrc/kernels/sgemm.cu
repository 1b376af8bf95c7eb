// fp32 GEMM on the CUDA cores: C[M,N] = A[M,K] * B[K,N], all row-major, fp32 multiply-add with fp32
// accumulation, optionally batched.  This is the full-precision path of CudaBackend.gemm_f32 /
// gemm_batched_f32: the tensor-core kernels of this library take bf16 operands, and an fp32 caller
// (the backend trait of the reference, crates/axonml-core/src/backends/cuda.rs:413-501, calls cuBLAS
// sgemm / sgemmStridedBatched) must not silently get bf16 products.
//
// 128 x 128 x 16 block tile, 256 threads with an 8 x 8 micro-tile each (two 4 x 4 quadrant pairs, so
// that the shared-memory reads of a warp are conflict-free float4 loads), operands staged through
// registers into double-buffered shared memory; A is stored transposed ([k][m]) so that both
// operands are read along their contiguous dimension in the inner loop.  Edges and unaligned
// leading dimensions take guarded scalar loads.
#include "common.cuh"

namespace {

constexpr int TM = 128, TN = 128, TK = 16;
constexpr int kThreads = 256;

struct SgemmParams {
  const float* A;
  const float* B;
  float* C;
  int M, N, K, lda, ldb, ldc;
  long sA, sB, sC;   // batch strides in elements
  int vec_ok;        // leading dimensions and base pointers allow float4 access
};

__global__ void __launch_bounds__(kThreads) sgemm_kernel(const SgemmParams p) {
  __shared__ __align__(16) float As[2][TK][TM + 4];
  __shared__ __align__(16) float Bs[2][TK][TN];
  const int tid = threadIdx.x;
  const float* A = p.A + (long)blockIdx.z * p.sA;
  const float* B = p.B + (long)blockIdx.z * p.sB;
  float* C = p.C + (long)blockIdx.z * p.sC;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;

  // loader coordinates: A: 2 float4 along k per thread; B: 2 float4 along n per thread
  const int a_row = tid >> 2, a_k = (tid & 3) * 4;        // rows a_row and a_row + 64
  const int b_k = tid >> 5, b_n = (tid & 31) * 4;         // k rows b_k and b_k + 8
  float4 ra[2], rb[2];

  auto load_tiles = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = m0 + a_row + 64 * i, k = k0 + a_k;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < p.M) {
        const float* src = A + (long)m * p.lda + k;
        if (p.vec_ok && k + 3 < p.K) {
          v = *reinterpret_cast<const float4*>(src);
        } else {
          if (k < p.K) v.x = src[0];
          if (k + 1 < p.K) v.y = src[1];
          if (k + 2 < p.K) v.z = src[2];
          if (k + 3 < p.K) v.w = src[3];
        }
      }
      ra[i] = v;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = k0 + b_k + 8 * i, n = n0 + b_n;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < p.K) {
        const float* src = B + (long)k * p.ldb + n;
        if (p.vec_ok && n + 3 < p.N) {
          v = *reinterpret_cast<const float4*>(src);
        } else {
          if (n < p.N) v.x = src[0];
          if (n + 1 < p.N) v.y = src[1];
          if (n + 2 < p.N) v.z = src[2];
          if (n + 3 < p.N) v.w = src[3];
        }
      }
      rb[i] = v;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = a_row + 64 * i;
      As[buf][a_k + 0][m] = ra[i].x;
      As[buf][a_k + 1][m] = ra[i].y;
      As[buf][a_k + 2][m] = ra[i].z;
      As[buf][a_k + 3][m] = ra[i].w;
      *reinterpret_cast<float4*>(&Bs[buf][b_k + 8 * i][b_n]) = rb[i];
    }
  };

  const int ty = tid >> 4, tx = tid & 15;   // micro-tile rows {4 ty .. +3, 64 + 4 ty .. +3}, cols likewise
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int num_k = (p.K + TK - 1) / TK;
  load_tiles(0);
  store_tiles(0);
  __syncthreads();
  for (int kt = 0; kt < num_k; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < num_k) load_tiles((kt + 1) * TK);
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < num_k) {
      store_tiles(buf ^ 1);     // the other buffer was last read before the previous barrier
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= p.M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + h * 64 + tx * 4;
      float* dst = C + (long)m * p.ldc + n;
      if (n >= p.N) continue;               // this thread's columns lie past the matrix
      if (!AX_INB((long)m * p.ldc + n, n + 3 < p.N ? 4 : p.N - n, (long)(p.M - 1) * p.ldc + p.N, 4000)) continue;
      if (p.vec_ok && n + 3 < p.N) {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) dst[j] = acc[i][4 * h + j];
      }
    }
  }
}

}  // namespace

// C[b] (fp32, [M,N], row stride ldc) = A[b] ([M,K], lda) * B[b] ([K,N], ldb) for b < batch; the
// batch strides are in elements (0 repeats an operand).  Returns a cudaError_t value or -1.
AX_API int ax_sgemm_f32(const float* A, const float* B, float* C, int M, int N, int K, int lda, int ldb,
                        int ldc, int batch, long strideA, long strideB, long strideC, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  if (K < 0 || lda < K || ldb < N || ldc < N || batch > 65535) return -1;
  SgemmParams p{A, B, C, M, N, K, lda, ldb, ldc, strideA, strideB, strideC, 0};
  p.vec_ok = ((lda | ldb | ldc) % 4 == 0) && (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) % 16 == 0) &&
             ((strideA | strideB | strideC) % 4 == 0);
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, batch);
  if (grid.y > 65535) return -1;
  sgemm_kernel<<<grid, kThreads, 0, stream>>>(p);
  return (int)cudaGetLastError();
}
