// CPU reference kernels (fp32, OpenMP): the numerical oracle for the CUDA kernels and a restatement
// of the reference's own CPU algorithms, which is also what its published CPU timings exercise
// (docs/index.md:124-133).  Covers CpuBackend (crates/axonml-core/src/backends/cpu.rs:137-731:
// elementwise, scalar ops, activations, reductions, matmul, transpose, dot, comparisons), the
// direct 7-loop convolution (crates/axonml-nn/src/layers/conv.rs:276-328), max pooling, row softmax,
// layer norm, inference batch norm, embedding gather and the attention-score product - i.e. the
// arithmetic of every WGSL/MSL compute shader of the reference (wgpu_backend.rs:1003-1603).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>

#define AX_API extern "C" __attribute__((visibility("default")))

namespace {
constexpr int64_t kParallelThreshold = 4096;   // cpu.rs:21
inline float gelu_tanh(float x) {
  return 0.5f * x * (1.f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
}  // namespace

// op: 0 add 1 sub 2 mul 3 div
AX_API void ax_cpu_binary(int op, const float* a, const float* b, float* y, int64_t n) {
#pragma omp parallel for if (n > kParallelThreshold)
  for (int64_t i = 0; i < n; ++i) {
    switch (op) {
      case 0: y[i] = a[i] + b[i]; break;
      case 1: y[i] = a[i] - b[i]; break;
      case 2: y[i] = a[i] * b[i]; break;
      default: y[i] = a[i] / b[i]; break;
    }
  }
}

// op: 0 neg 1 abs 2 relu 3 sigmoid 4 tanh 5 exp 6 ln 7 sqrt 8 square 9 gelu 10 silu 11 add_scalar 12 mul_scalar
//     13 leaky_relu(p) 14 elu(p)
AX_API void ax_cpu_unary(int op, const float* x, float* y, int64_t n, float p) {
#pragma omp parallel for if (n > kParallelThreshold)
  for (int64_t i = 0; i < n; ++i) {
    const float v = x[i];
    float r;
    switch (op) {
      case 0: r = -v; break;
      case 1: r = std::fabs(v); break;
      case 2: r = v > 0 ? v : 0; break;
      case 3: r = 1.f / (1.f + std::exp(-v)); break;
      case 4: r = std::tanh(v); break;
      case 5: r = std::exp(v); break;
      case 6: r = std::log(v); break;
      case 7: r = std::sqrt(v); break;
      case 8: r = v * v; break;
      case 9: r = gelu_tanh(v); break;
      case 10: r = v / (1.f + std::exp(-v)); break;
      case 11: r = v + p; break;
      case 12: r = v * p; break;
      case 13: r = v > 0 ? v : p * v; break;
      default: r = v > 0 ? v : p * (std::exp(v) - 1.f); break;
    }
    y[i] = r;
  }
}

// op: 0 sum 1 prod 2 max 3 min 4 mean 5 argmax 6 argmin (result as double)
AX_API double ax_cpu_reduce(int op, const float* x, int64_t n) {
  if (n <= 0) return 0.0;
  if (op == 0 || op == 4) {
    double s = 0;
#pragma omp parallel for reduction(+ : s) if (n > kParallelThreshold)
    for (int64_t i = 0; i < n; ++i) s += x[i];
    return op == 4 ? s / (double)n : s;
  }
  if (op == 1) {
    double p = 1;
    for (int64_t i = 0; i < n; ++i) p *= x[i];
    return p;
  }
  int64_t best = 0;
  for (int64_t i = 1; i < n; ++i) {
    const bool better = (op == 2 || op == 5) ? x[i] > x[best] : x[i] < x[best];
    if (better) best = i;
  }
  return (op == 5 || op == 6) ? (double)best : (double)x[best];
}

AX_API double ax_cpu_dot(const float* a, const float* b, int64_t n) {
  double s = 0;
#pragma omp parallel for reduction(+ : s) if (n > kParallelThreshold)
  for (int64_t i = 0; i < n; ++i) s += (double)a[i] * b[i];
  return s;
}

// C[M,N] = A[M,K] * B[K,N], row-major, cache-blocked (tile 64 as in the reference's fallback)
AX_API void ax_cpu_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  constexpr int64_t T = 64;
  memset(C, 0, sizeof(float) * M * N);
#pragma omp parallel for schedule(static)
  for (int64_t i0 = 0; i0 < M; i0 += T)
    for (int64_t k0 = 0; k0 < K; k0 += T)
      for (int64_t j0 = 0; j0 < N; j0 += T) {
        const int64_t i1 = std::min(i0 + T, M), k1 = std::min(k0 + T, K), j1 = std::min(j0 + T, N);
        for (int64_t i = i0; i < i1; ++i)
          for (int64_t k = k0; k < k1; ++k) {
            const float a = A[i * K + k];
            const float* b = B + k * N;
            float* c = C + i * N;
            for (int64_t j = j0; j < j1; ++j) c[j] += a * b[j];
          }
      }
}

AX_API void ax_cpu_transpose(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for if (rows * cols > kParallelThreshold)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) y[c * rows + r] = x[r * cols + c];
}

// op: 0 eq 1 lt 2 gt -> 1.0 / 0.0
AX_API void ax_cpu_compare(int op, const float* a, const float* b, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = (op == 0 ? a[i] == b[i] : op == 1 ? a[i] < b[i] : a[i] > b[i]) ? 1.f : 0.f;
}

// direct NCHW convolution with bias, stride and zero padding
AX_API void ax_cpu_conv2d(const float* x, const float* w, const float* bias, float* y, int N, int C,
                          int H, int W, int O, int KH, int KW, int SH, int SW, int PH, int PW) {
  const int OH = (H + 2 * PH - KH) / SH + 1, OW = (W + 2 * PW - KW) / SW + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int o = 0; o < O; ++o)
      for (int oh = 0; oh < OH; ++oh)
        for (int ow = 0; ow < OW; ++ow) {
          float acc = bias ? bias[o] : 0.f;
          for (int c = 0; c < C; ++c)
            for (int kh = 0; kh < KH; ++kh) {
              const int ih = oh * SH - PH + kh;
              if (ih < 0 || ih >= H) continue;
              for (int kw = 0; kw < KW; ++kw) {
                const int iw = ow * SW - PW + kw;
                if (iw < 0 || iw >= W) continue;
                acc += x[((int64_t)(n * C + c) * H + ih) * W + iw] * w[((int64_t)(o * C + c) * KH + kh) * KW + kw];
              }
            }
          y[((int64_t)(n * O + o) * OH + oh) * OW + ow] = acc;
        }
}

AX_API void ax_cpu_maxpool2d(const float* x, float* y, int NC, int H, int W, int K, int S, int P) {
  const int OH = (H + 2 * P - K) / S + 1, OW = (W + 2 * P - K) / S + 1;
#pragma omp parallel for schedule(static)
  for (int nc = 0; nc < NC; ++nc)
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        float m = -INFINITY;
        for (int kh = 0; kh < K; ++kh)
          for (int kw = 0; kw < K; ++kw) {
            const int ih = oh * S - P + kh, iw = ow * S - P + kw;
            if (ih >= 0 && ih < H && iw >= 0 && iw < W) m = std::max(m, x[((int64_t)nc * H + ih) * W + iw]);
          }
        y[((int64_t)nc * OH + oh) * OW + ow] = m;
      }
}

AX_API void ax_cpu_softmax_rows(const float* x, float* y, int64_t rows, int64_t cols, int log_mode) {
#pragma omp parallel for if (rows * cols > kParallelThreshold)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    float m = -INFINITY;
    for (int64_t c = 0; c < cols; ++c) m = std::max(m, xr[c]);
    double s = 0;
    for (int64_t c = 0; c < cols; ++c) s += std::exp((double)xr[c] - m);
    const float lse = m + (float)std::log(s);
    for (int64_t c = 0; c < cols; ++c) yr[c] = log_mode ? xr[c] - lse : std::exp(xr[c] - lse);
  }
}

AX_API void ax_cpu_layer_norm(const float* x, const float* w, const float* b, float* y, int64_t rows,
                              int64_t D, float eps, int rms) {
#pragma omp parallel for if (rows * D > kParallelThreshold)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * D;
    double s = 0, ss = 0;
    for (int64_t c = 0; c < D; ++c) { s += xr[c]; ss += (double)xr[c] * xr[c]; }
    const double mean = rms ? 0.0 : s / D;
    const double var = rms ? ss / D : std::max(ss / D - mean * mean, 0.0);
    const float rstd = (float)(1.0 / std::sqrt(var + eps));
    for (int64_t c = 0; c < D; ++c)
      y[r * D + c] = (xr[c] - (float)mean) * rstd * (w ? w[c] : 1.f) + (b ? b[c] : 0.f);
  }
}

// inference batch norm on NCHW with running statistics
AX_API void ax_cpu_batch_norm(const float* x, const float* mean, const float* var, const float* w,
                              const float* b, float* y, int N, int C, int64_t HW, float eps) {
#pragma omp parallel for collapse(2)
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      const float sc = (w ? w[c] : 1.f) / std::sqrt(var[c] + eps), sh = (b ? b[c] : 0.f) - mean[c] * sc;
      const int64_t base = ((int64_t)n * C + c) * HW;
      for (int64_t i = 0; i < HW; ++i) y[base + i] = x[base + i] * sc + sh;
    }
}

AX_API void ax_cpu_embedding(const int64_t* idx, const float* W, float* y, int64_t n, int64_t D, int64_t V) {
#pragma omp parallel for if (n * D > kParallelThreshold)
  for (int64_t i = 0; i < n; ++i) {
    if (idx[i] >= 0 && idx[i] < V) memcpy(y + i * D, W + idx[i] * D, sizeof(float) * D);
    else memset(y + i * D, 0, sizeof(float) * D);
  }
}

// scores[b,h,q,k] = scale * sum_d Q[b,h,q,d] K[b,h,k,d]
AX_API void ax_cpu_attention_scores(const float* Q, const float* K, float* S, int BH, int Sq, int Sk,
                                    int D, float scale) {
#pragma omp parallel for collapse(2)
  for (int bh = 0; bh < BH; ++bh)
    for (int q = 0; q < Sq; ++q)
      for (int k = 0; k < Sk; ++k) {
        double acc = 0;
        for (int d = 0; d < D; ++d) acc += (double)Q[((int64_t)bh * Sq + q) * D + d] * K[((int64_t)bh * Sk + k) * D + d];
        S[((int64_t)bh * Sq + q) * Sk + k] = (float)acc * scale;
      }
}

// blockwise ("flash") attention forward on the CPU, [BH, S, D], online softmax, block 64
// (same algorithm as crates/axonml-llm/src/attention.rs:836-943)
AX_API void ax_cpu_flash_attention(const float* Q, const float* K, const float* V, float* O, int BH,
                                   int Sq, int Sk, int D, float scale, int causal, int block) {
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < BH; ++bh)
    for (int q = 0; q < Sq; ++q) {
      float m = -INFINITY;
      double l = 0;
      float* o = O + ((int64_t)bh * Sq + q) * D;
      for (int d = 0; d < D; ++d) o[d] = 0;
      const int limit = causal ? std::min(Sk - 1, q + (Sk - Sq)) : Sk - 1;
      for (int k0 = 0; k0 <= limit; k0 += block) {
        const int k1 = std::min(k0 + block, limit + 1);
        float bm = -INFINITY;
        float s[256];
        for (int k = k0; k < k1; ++k) {
          double acc = 0;
          for (int d = 0; d < D; ++d) acc += (double)Q[((int64_t)bh * Sq + q) * D + d] * K[((int64_t)bh * Sk + k) * D + d];
          s[k - k0] = (float)acc * scale;
          bm = std::max(bm, s[k - k0]);
        }
        const float mn = std::max(m, bm);
        const float alpha = std::exp(m - mn);
        l *= alpha;
        for (int d = 0; d < D; ++d) o[d] *= alpha;
        for (int k = k0; k < k1; ++k) {
          const float p = std::exp(s[k - k0] - mn);
          l += p;
          const float* v = V + ((int64_t)bh * Sk + k) * D;
          for (int d = 0; d < D; ++d) o[d] += p * v[d];
        }
        m = mn;
      }
      const float inv = l > 0 ? (float)(1.0 / l) : 0.f;
      for (int d = 0; d < D; ++d) o[d] *= inv;
    }
}
