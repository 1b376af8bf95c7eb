// Multi-tensor fused optimizers.  One launch updates up to kMaxTensors tensors: the kernel
// parameters carry a table of tensor pointers and a block -> (tensor, chunk) map, so that a whole
// model is stepped in a handful of launches instead of several per parameter.
//
// Every update can (a) multiply the gradient by a device-resident 1/loss-scale, (b) skip itself
// when a device-resident found-inf flag is set (GradScaler semantics without a host sync), and
// (c) write a bf16 copy of the updated fp32 master parameter.
//
// Update rules follow the reference: SGD crates/axonml-optim/src/sgd.rs:132-198, Adam/AdamW
// adam.rs:158-234 and :376-445, RMSprop rmsprop.rs:181-250, LAMB lamb.rs:200-280, gradient
// clipping crates/axonml/src/trainer.rs:413-440, GradScaler unscale grad_scaler.rs:187-206.
#include "common.cuh"

namespace {
using namespace ax;

constexpr int kMaxTensors = 24;
constexpr int kMaxBlocks = 1 << 20;  // blocks of one launch (a grid-size bound, not a table size)
constexpr int kChunk = 2048 * 32;    // elements per block

struct TensorTable {
  void* p[kMaxTensors];    // parameter (fp32 or bf16)
  void* g[kMaxTensors];    // gradient (fp32 or bf16)
  float* s1[kMaxTensors];  // state 1 (momentum / exp_avg / square_avg)
  float* s2[kMaxTensors];  // state 2 (exp_avg_sq / momentum buffer)
  float* s3[kMaxTensors];  // state 3 (amsgrad max / grad_avg / LAMB update)
  __nv_bfloat16* lp[kMaxTensors];  // optional low-precision copy of p
  long n[kMaxTensors];
  int gidx[kMaxTensors];  // index of the tensor in the caller's list (for per-tensor norms)
  // Block b works on chunk (b - first_blk[t]) of the tensor t with first_blk[t] <= b < first_blk[t+1].
  // A cumulative table keeps the launch independent of the number of blocks: one launch covers
  // whole tensors, and the grid has thousands of blocks instead of a 320-entry block table whose
  // 2.2 blocks per SM left a quarter of the machine idle in the last round.
  int first_blk[kMaxTensors + 1];
  int chunk0[kMaxTensors];   // first chunk of the tensor handled by this launch
  int num;
};

struct Hyper {
  float lr, beta1, beta2, eps, wd, bc1, bc2;  // bc = 1 - beta^t
  float momentum, dampening, alpha;
  int nesterov, first_step, adamw, amsgrad, centered;
  const float* inv_scale;  // may be null
  const int* found_inf;    // may be null: skip everything when *found_inf != 0
  float* norms;            // LAMB: [tensor][2] sums of squares; grad-norm: [1]
  const float* clip_coef;  // optional device scalar multiplied into the gradient
  const int* step_dev;     // optional: steps taken so far, kept on the device; when given, the bias
                           // corrections are 1 - beta^(*step_dev + 1) and bc1 / bc2 are ignored (the
                           // host cannot know how many steps a device-side found-inf flag skipped)
};

template <typename T> __device__ __forceinline__ float ld(const T* p, long i);
template <> __device__ __forceinline__ float ld<float>(const float* p, long i) { return p[i]; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void st(T* p, long i, float v);
template <> __device__ __forceinline__ void st<float>(float* p, long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, long i, float v) { p[i] = __float2bfloat16(v); }

__device__ __forceinline__ void ld4(const float* p, long i, float (&v)[4]) {
  float4 t = *reinterpret_cast<const float4*>(p + i);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, long i, float (&v)[4]) {
  uint2 t = *reinterpret_cast<const uint2*>(p + i);
  float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void st4(float* p, long i, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, long i, const float (&v)[4]) {
  uint2 t;
  t.x = pack_bf16x2(v[0], v[1]); t.y = pack_bf16x2(v[2], v[3]);
  *reinterpret_cast<uint2*>(p + i) = t;
}

enum Kind : int { K_SGD = 0, K_ADAM, K_RMSPROP, K_LAMB1, K_LAMB2, K_SUMSQ, K_SCALE, K_UNSCALE_CHECK };

template <int KIND, typename PT, typename GT>
__global__ void __launch_bounds__(512)
mt_kernel(const TensorTable tt, const Hyper h_in) {
  Hyper h = h_in;
  if (KIND != K_SUMSQ && KIND != K_UNSCALE_CHECK && h.found_inf && *h.found_inf) return;
  int t = 0;
  while (t + 1 < tt.num && (int)blockIdx.x >= tt.first_blk[t + 1]) ++t;
  const long base = (long)(tt.chunk0[t] + (int)blockIdx.x - tt.first_blk[t]) * kChunk;
  const long n = tt.n[t];
  const long end = base + kChunk < n ? base + kChunk : n;
  PT* p = (PT*)tt.p[t];
  GT* g = (GT*)tt.g[t];
  float* s1 = tt.s1[t];
  float* s2 = tt.s2[t];
  float* s3 = tt.s3[t];
  __nv_bfloat16* lp = tt.lp[t];
  float gmul = h.inv_scale ? *h.inv_scale : 1.f;
  if (h.clip_coef) gmul *= *h.clip_coef;
  if ((KIND == K_ADAM || KIND == K_LAMB1) && h.step_dev != nullptr && h.bc1 != 1.f) {
    const double t = (double)(*h.step_dev + 1);
    h.bc1 = (float)(1.0 - pow((double)h.beta1, t));
    h.bc2 = (float)(1.0 - pow((double)h.beta2, t));
  }
  float acc0 = 0.f, acc1 = 0.f;
  int bad = 0;
  float trust = 1.f;
  if (KIND == K_LAMB2) {
    float pn = sqrtf(h.norms[2 * tt.gidx[t]]), rn = sqrtf(h.norms[2 * tt.gidx[t] + 1]);
    trust = (pn > 0.f && rn > 0.f) ? pn / rn : 1.f;
  }
  // One element of the update.  w: parameter, gr: raw gradient, a/b/c: optimizer states.
  auto elem = [&](float& w, float& gr, float& a, float& b, float& c) {
    if (KIND == K_SGD) {
      gr = gr * gmul + h.wd * w;
      if (h.momentum != 0.f) {
        a = h.first_step ? gr : h.momentum * a + (1.f - h.dampening) * gr;
        gr = h.nesterov ? gr + h.momentum * a : a;
      }
      w -= h.lr * gr;
    } else if (KIND == K_ADAM) {
      gr *= gmul;
      if (h.adamw) w *= 1.f - h.lr * h.wd; else gr += h.wd * w;
      a = h.beta1 * a + (1.f - h.beta1) * gr;
      b = h.beta2 * b + (1.f - h.beta2) * gr * gr;
      float vv = b;
      if (h.amsgrad) { vv = fmaxf(c, b); c = vv; }
      w -= (h.lr / h.bc1) * a / (sqrtf(vv / h.bc2) + h.eps);
    } else if (KIND == K_RMSPROP) {
      gr = gr * gmul + h.wd * w;
      a = h.alpha * a + (1.f - h.alpha) * gr * gr;
      float avg;
      if (h.centered) {
        c = h.alpha * c + (1.f - h.alpha) * gr;
        avg = sqrtf(fmaxf(a - c * c, 0.f)) + h.eps;
      } else {
        avg = sqrtf(a) + h.eps;
      }
      if (h.momentum > 0.f) {
        b = h.momentum * b + gr / avg;
        w -= h.lr * b;
      } else {
        w -= h.lr * gr / avg;
      }
    } else if (KIND == K_LAMB1) {
      gr *= gmul;
      a = h.beta1 * a + (1.f - h.beta1) * gr;
      b = h.beta2 * b + (1.f - h.beta2) * gr * gr;
      c = (a / h.bc1) / (sqrtf(b / h.bc2) + h.eps) + h.wd * w;
      acc0 += w * w;
      acc1 += c * c;
    } else if (KIND == K_LAMB2) {
      w -= h.lr * trust * c;
    } else if (KIND == K_SUMSQ) {
      gr *= gmul;
      acc0 += gr * gr;
    } else if (KIND == K_SCALE) {
      gr *= gmul;
    } else if (KIND == K_UNSCALE_CHECK) {
      gr *= gmul;
      if (!isfinite(gr)) bad = 1;
    }
  };
  constexpr bool kUsesP = KIND == K_SGD || KIND == K_ADAM || KIND == K_RMSPROP || KIND == K_LAMB1 || KIND == K_LAMB2;
  constexpr bool kWritesP = KIND == K_SGD || KIND == K_ADAM || KIND == K_RMSPROP || KIND == K_LAMB2;
  constexpr bool kUsesG = KIND != K_LAMB2;
  constexpr bool kWritesG = KIND == K_SCALE || KIND == K_UNSCALE_CHECK;
  constexpr bool kS1 = KIND == K_SGD || KIND == K_ADAM || KIND == K_RMSPROP || KIND == K_LAMB1;
  constexpr bool kS2 = KIND == K_ADAM || KIND == K_RMSPROP || KIND == K_LAMB1;
  constexpr bool kS3R = KIND == K_ADAM || KIND == K_RMSPROP || KIND == K_LAMB2;
  constexpr bool kS3W = KIND == K_ADAM || KIND == K_RMSPROP || KIND == K_LAMB1;
  const bool use_s1 = kS1 && s1 != nullptr && !(KIND == K_SGD && h.momentum == 0.f);
  const bool use_s2 = kS2 && s2 != nullptr && !(KIND == K_RMSPROP && h.momentum <= 0.f);
  const bool use_s3 = s3 != nullptr && ((KIND == K_ADAM && h.amsgrad) || (KIND == K_RMSPROP && h.centered) ||
                                        KIND == K_LAMB1 || KIND == K_LAMB2);
  // vector path: 4 elements per thread per iteration when every pointer is 16-byte aligned
  const uintptr_t al = (kUsesP ? (uintptr_t)p : 0) | (kUsesG ? (uintptr_t)g : 0) | (use_s1 ? (uintptr_t)s1 : 0) |
                       (use_s2 ? (uintptr_t)s2 : 0) | (use_s3 ? (uintptr_t)s3 : 0) | (uintptr_t)lp;
  const bool vec = (al & 15) == 0;
  const long vend = vec ? base + ((end - base) & ~3L) : base;
  for (long i = base + threadIdx.x * 4L; i < vend; i += blockDim.x * 4L) {
    float w[4] = {0, 0, 0, 0}, gr[4] = {0, 0, 0, 0}, a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0}, c[4] = {0, 0, 0, 0};
    if (kUsesP) ld4(p, i, w);
    if (kUsesG) ld4(g, i, gr);
    if (use_s1) ld4(s1, i, a);
    if (use_s2) ld4(s2, i, b);
    if (use_s3 && kS3R) ld4(s3, i, c);
#pragma unroll
    for (int j = 0; j < 4; ++j) elem(w[j], gr[j], a[j], b[j], c[j]);
    if (kWritesP) { st4(p, i, w); if (lp) st4(lp, i, w); }
    if (kWritesG) st4(g, i, gr);
    if (use_s1) st4(s1, i, a);
    if (use_s2) st4(s2, i, b);
    if (use_s3 && kS3W) st4(s3, i, c);
  }
  for (long i = vend + threadIdx.x; i < end; i += blockDim.x) {
    float w = kUsesP ? ld(p, i) : 0.f, gr = kUsesG ? ld(g, i) : 0.f;
    float a = use_s1 ? s1[i] : 0.f, b = use_s2 ? s2[i] : 0.f, c = (use_s3 && kS3R) ? s3[i] : 0.f;
    elem(w, gr, a, b, c);
    if (kWritesP) { st(p, i, w); if (lp) lp[i] = __float2bfloat16(w); }
    if (kWritesG) st(g, i, gr);
    if (use_s1) s1[i] = a;
    if (use_s2) s2[i] = b;
    if (use_s3 && kS3W) s3[i] = c;
  }
  if (KIND == K_LAMB1 || KIND == K_SUMSQ) {
    __shared__ float r0[16], r1[16];
    acc0 = warp_sum(acc0);
    acc1 = warp_sum(acc1);
    if ((threadIdx.x & 31) == 0) { r0[threadIdx.x >> 5] = acc0; r1[threadIdx.x >> 5] = acc1; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.f, b = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { a += r0[w]; b += r1[w]; }
      if (KIND == K_LAMB1) {
        atomicAdd(&h.norms[2 * tt.gidx[t]], a);
        atomicAdd(&h.norms[2 * tt.gidx[t] + 1], b);
      } else {
        atomicAdd(&h.norms[0], a);
      }
    }
  }
  if (KIND == K_UNSCALE_CHECK) {
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch((int*)h.norms, 1);
  }
}

template <int KIND>
int launch_typed(int p_bf16, int g_bf16, const TensorTable& tt, const Hyper& h, int blocks,
                 cudaStream_t stream) {
  if (!p_bf16 && !g_bf16) mt_kernel<KIND, float, float><<<blocks, 512, 0, stream>>>(tt, h);
  else if (!p_bf16 && g_bf16) mt_kernel<KIND, float, __nv_bfloat16><<<blocks, 512, 0, stream>>>(tt, h);
  else if (p_bf16 && g_bf16) mt_kernel<KIND, __nv_bfloat16, __nv_bfloat16><<<blocks, 512, 0, stream>>>(tt, h);
  else mt_kernel<KIND, __nv_bfloat16, float><<<blocks, 512, 0, stream>>>(tt, h);
  return (int)cudaGetLastError();
}

}  // namespace

// Generic entry: `kind` selects the update (see Kind).  Pointer arrays have `nt` entries (entries
// of unused state arrays may be null).  hyper: float[10] = lr, beta1, beta2, eps, wd, bc1, bc2,
// momentum, dampening, alpha; flags: int[5] = nesterov, first_step, adamw, amsgrad, centered.
AX_API int ax_multi_tensor(int kind, int p_bf16, int g_bf16, int nt, void** p, void** g, void** s1,
                           void** s2, void** s3, void** lp, const long* n, const float* hyper,
                           const int* flags, const float* inv_scale, const int* found_inf,
                           float* norms, const float* clip_coef, const int* step_dev, cudaStream_t stream) {
  Hyper h;
  h.lr = hyper[0]; h.beta1 = hyper[1]; h.beta2 = hyper[2]; h.eps = hyper[3]; h.wd = hyper[4];
  h.bc1 = hyper[5]; h.bc2 = hyper[6]; h.momentum = hyper[7]; h.dampening = hyper[8]; h.alpha = hyper[9];
  h.nesterov = flags[0]; h.first_step = flags[1]; h.adamw = flags[2]; h.amsgrad = flags[3]; h.centered = flags[4];
  h.inv_scale = inv_scale; h.found_inf = found_inf; h.norms = norms; h.clip_coef = clip_coef;
  h.step_dev = step_dev;

  TensorTable tt;
  int nt_in = 0, nb = 0, rc = 0;
  auto flush = [&]() {
    if (nb == 0) return 0;
    int r;
    switch (kind) {
      case K_SGD: r = launch_typed<K_SGD>(p_bf16, g_bf16, tt, h, nb, stream); break;
      case K_ADAM: r = launch_typed<K_ADAM>(p_bf16, g_bf16, tt, h, nb, stream); break;
      case K_RMSPROP: r = launch_typed<K_RMSPROP>(p_bf16, g_bf16, tt, h, nb, stream); break;
      case K_LAMB1: r = launch_typed<K_LAMB1>(p_bf16, g_bf16, tt, h, nb, stream); break;
      case K_LAMB2: r = launch_typed<K_LAMB2>(p_bf16, g_bf16, tt, h, nb, stream); break;
      case K_SUMSQ: r = launch_typed<K_SUMSQ>(p_bf16, g_bf16, tt, h, nb, stream); break;
      case K_SCALE: r = launch_typed<K_SCALE>(p_bf16, g_bf16, tt, h, nb, stream); break;
      case K_UNSCALE_CHECK: r = launch_typed<K_UNSCALE_CHECK>(p_bf16, g_bf16, tt, h, nb, stream); break;
      default: r = -1;
    }
    nb = 0;
    return r;
  };
  for (int t = 0; t < nt; ++t) {
    if (n[t] <= 0) continue;
    const long chunks = (n[t] + kChunk - 1) / kChunk;
    long c = 0;
    while (c < chunks) {
      if (nt_in == kMaxTensors || nb == kMaxBlocks) {
        if ((rc = flush())) return rc;
        nt_in = 0;
      }
      const int slot = nt_in++;
      tt.p[slot] = p ? p[t] : nullptr;
      tt.g[slot] = g ? g[t] : nullptr;
      tt.s1[slot] = s1 ? (float*)s1[t] : nullptr;
      tt.s2[slot] = s2 ? (float*)s2[t] : nullptr;
      tt.s3[slot] = s3 ? (float*)s3[t] : nullptr;
      tt.lp[slot] = lp ? (__nv_bfloat16*)lp[t] : nullptr;
      tt.n[slot] = n[t];
      tt.gidx[slot] = t;
      const int take = (int)((chunks - c) < (long)(kMaxBlocks - nb) ? (chunks - c) : (long)(kMaxBlocks - nb));
      tt.first_blk[slot] = nb;
      tt.chunk0[slot] = (int)c;
      nb += take;
      c += take;
      tt.first_blk[slot + 1] = nb;
      tt.num = slot + 1;
    }
  }
  return flush();
}

AX_API int ax_multi_tensor_limits(int* max_tensors, int* max_blocks, int* chunk) {
  *max_tensors = kMaxTensors; *max_blocks = kMaxBlocks; *chunk = kChunk;
  return 0;
}
