// Paged KV cache for serving: a write kernel that scatters new K/V rows into cache pages and the
// decode attention kernel (one query token per sequence) that reads K/V through a block table.
//
// Cache layout: k_cache / v_cache [num_pages, page_size, Hkv, D] bf16; block_table [B, max_pages]
// int32; context_lens [B] int32.  Grouped-query attention: the G = Hq/Hkv query heads that share
// a KV head are processed by the same CTA, so each K/V row is read once for all of them.
// One CTA per (sequence, kv head, split of the context); 8 lanes cooperate on a token (each holds
// 16 elements of the row), so a warp covers 4 tokens per iteration with 16-byte loads; every
// 8-lane group keeps its own online softmax state; groups are merged with shuffles, warps through
// shared memory, context splits by a small second kernel.
//
// Replaces the reference's concat-and-grow KVCache (crates/axonml-llm/src/attention.rs:46-70) and
// the full score-matrix attention of crates/axonml-llm/src/llama.rs:429-441 for the decode step.
#include "common.cuh"

namespace {
using namespace ax;

constexpr int kWarps = 8;
constexpr int kLanesPerTok = 8;                       // lanes that share one cached token
constexpr int kTokPerWarp = 32 / kLanesPerTok;
constexpr int kTokPerIter = kWarps * kTokPerWarp;     // tokens a CTA covers per iteration
constexpr int D = 128;
constexpr int kEl = D / kLanesPerTok;                 // 16 elements of a row per lane
constexpr int kMaxG = 8;                              // query heads per KV head handled in one pass

__global__ void paged_kv_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                      __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                      const int* __restrict__ block_table, const int* __restrict__ seq_ids,
                                      const int* __restrict__ positions, int tokens, int row_elems,
                                      long k_stride, long v_stride, int page_size, int max_pages) {
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const int b = seq_ids[t], pos = positions[t];
    const int page = block_table[b * max_pages + pos / page_size];
    const long dst = ((long)page * page_size + pos % page_size) * row_elems;
    for (int i = threadIdx.x * 8; i < row_elems; i += blockDim.x * 8) {
      *reinterpret_cast<uint4*>(kc + dst + i) = *reinterpret_cast<const uint4*>(k + t * k_stride + i);
      *reinterpret_cast<uint4*>(vc + dst + i) = *reinterpret_cast<const uint4*>(v + t * v_stride + i);
    }
  }
}

// Unpacks 8 bf16 (one 16-byte load) into floats.
__device__ __forceinline__ void unpack8(const uint4 u, float* d) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
  d[0] = a.x; d[1] = a.y; d[2] = b.x; d[3] = b.y; d[4] = c.x; d[5] = c.y; d[6] = e.x; d[7] = e.y;
}

// Grid (B, Hkv, S): split s of sequence b covers an equal share of the sequence's tokens (rounded
// up to the 32 tokens a CTA handles per iteration), so one query token still fills the GPU.  With
// S == 1 the result goes straight to `out`; otherwise un-normalised partial sums and (max, sum)
// go to `part` [B, Hq, S, D + 2] fp32 and paged_merge_kernel finishes.
template <int G>
__global__ void __launch_bounds__(kWarps * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out,
                    float* __restrict__ part, const int* __restrict__ block_table,
                    const int* __restrict__ ctx_lens, int Hq, int Hkv, int page_size, int max_pages,
                    float scale_log2, long q_stride, long o_stride) {
  const int b = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z, S = gridDim.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & (kLanesPerTok - 1);     // which 16 elements of the row this lane holds
  const int slot = warp * kTokPerWarp + lane / kLanesPerTok;
  const int ctx = ctx_lens[b];
  const int chunk = (((ctx + S - 1) / S) + kTokPerIter - 1) / kTokPerIter * kTokPerIter;
  const int t_begin = sp * chunk;
  const int t_end = min(ctx, t_begin + chunk);
  const int h0 = hk * G;
  float qv[G][kEl];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q + (long)b * q_stride + (long)(h0 + g) * D + sub * kEl;
    unpack8(*reinterpret_cast<const uint4*>(qp), &qv[g][0]);
    unpack8(*reinterpret_cast<const uint4*>(qp + 8), &qv[g][8]);
  }
  float m[G], l[G], acc[G][kEl];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < kEl; ++i) acc[g][i] = 0.f;
  }
  const long row = (long)Hkv * D;
  // The K/V rows of the next 32 tokens are requested before the current ones are used, so that
  // two iterations of loads are in flight per thread.
  uint4 nk0, nk1, nv0, nv1;
  bool nvalid = false;
  auto issue = [&](int t0) {
    const int t = t0 + slot;
    nvalid = t < t_end;
    if (nvalid) {
      const int page = block_table[b * max_pages + t / page_size];
      const long off = ((long)page * page_size + t % page_size) * row + (long)hk * D + sub * kEl;
      nk0 = *reinterpret_cast<const uint4*>(kc + off); nk1 = *reinterpret_cast<const uint4*>(kc + off + 8);
      nv0 = *reinterpret_cast<const uint4*>(vc + off); nv1 = *reinterpret_cast<const uint4*>(vc + off + 8);
    }
  };
  if (t_begin < t_end) issue(t_begin);
  for (int t0 = t_begin; t0 < t_end; t0 += kTokPerIter) {
    const bool valid = nvalid;
    const uint4 k0 = nk0, k1 = nk1, v0 = nv0, v1 = nv1;
    if (t0 + kTokPerIter < t_end) issue(t0 + kTokPerIter);
    float kf[kEl], vf[kEl];
    if (valid) {
      unpack8(k0, kf); unpack8(k1, kf + 8);
      unpack8(v0, vf); unpack8(v1, vf + 8);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
      if (valid) {
#pragma unroll
        for (int i = 0; i < kEl; ++i) s += qv[g][i] * kf[i];
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (valid) {
        s *= scale_log2;
        const float mn = fmaxf(m[g], s);
        const float alpha = exp2f(m[g] - mn), pe = exp2f(s - mn);
        l[g] = l[g] * alpha + pe;
#pragma unroll
        for (int i = 0; i < kEl; ++i) acc[g][i] = acc[g][i] * alpha + pe * vf[i];
        m[g] = mn;
      }
    }
  }
  // merge the token slots of a warp with shuffles, then the warps through shared memory
  __shared__ float sM[kMaxG][kWarps], sL[kMaxG][kWarps];
  __shared__ float sO[kWarps][G][D];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = fmaxf(m[g], __shfl_xor_sync(0xffffffffu, m[g], 8));
    M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 16));
    const float w = m[g] == -INFINITY ? 0.f : exp2f(m[g] - M);
    float L = l[g] * w;
    L += __shfl_xor_sync(0xffffffffu, L, 8);
    L += __shfl_xor_sync(0xffffffffu, L, 16);
#pragma unroll
    for (int i = 0; i < kEl; ++i) {
      float a = acc[g][i] * w;
      a += __shfl_xor_sync(0xffffffffu, a, 8);
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      if (lane < kLanesPerTok) sO[warp][g][sub * kEl + i] = a;
    }
    if (lane == 0) { sM[g][warp] = M; sL[g][warp] = L; }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, sM[g][w]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = sM[g][w] == -INFINITY ? 0.f : exp2f(sM[g][w] - M);
      L += sL[g][w] * f;
      O += sO[w][g][d] * f;
    }
    if (S == 1) {
      out[(long)b * o_stride + (long)(h0 + g) * D + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
    } else {
      float* pp = part + (((long)b * Hq + h0 + g) * S + sp) * (D + 2);
      pp[d] = O;
      if (d == 0) { pp[D] = M; pp[D + 1] = L; }
    }
  }
}

constexpr int kTPage = 16;        // page size of the tensor-core decode path

// ---------------------------------------------------------------------------------------------
// Decode attention on the warp-level tensor-core path (mma.sync m16n8k16, bf16 in, fp32 out).
// With grouped-query attention the G query heads that share a KV head form the rows of a small
// matrix: S[G x 16] = Q[G x 128] K_page^T and O[G x 128] += P[G x 16] V_page per 16-token page.
// On CUDA cores those products cost 2 FMAs per byte of KV cache, which caps the kernel near a
// quarter of HBM speed; as MMAs (rows padded to 16) they are a handful of instructions per page.
// A producer warp keeps kMStages pages in flight with TMA (per page: K and V, each as two
// 64-dim halves in the 128-byte swizzle so that ldmatrix is conflict-free); four consumer warps
// take pages round-robin, each with its own online-softmax state, and merge at the end.
constexpr int kMWarps = 4;
constexpr int kMStages = 8;
constexpr int kMHalf = kTPage * 64 * 2;            // 2 KB: 16 tokens x 64 dims
constexpr int kMStageBytes = 4 * kMHalf;           // K lo, K hi, V lo, V hi

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int G>
__global__ void __launch_bounds__((kMWarps + 1) * 32)
paged_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, float* __restrict__ part,
                        const int* __restrict__ block_table, const int* __restrict__ ctx_lens, int Hq, int Hkv,
                        int max_pages, float scale_log2, long q_stride, long o_stride, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + kMStages * kMStageBytes);
  uint64_t* empty = full + kMStages;
  volatile int* dead = (volatile int*)(empty + kMStages);
  float* sM = (float*)(dead + 2);                       // [G][warps]
  float* sL = sM + kMaxG * kMWarps;
  float* sO = sL + kMaxG * kMWarps;                     // [warps][G][D]

  const int b = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z, S = gridDim.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ctx = ctx_lens[b];
  const int pages = (ctx + kTPage - 1) / kTPage;
  const int per = (pages + S - 1) / S;
  const int p_begin = sp * per, p_end = min(pages, p_begin + per);
  const int h0 = hk * G;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < kMStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    mbar_fence_init();
  }
  __syncthreads();

  const int grow = lane >> 2;             // row of the 16 x N fragments this lane holds = query head
  const int qcol = (lane & 3) * 2;        // first of its two columns inside an 8-wide tile
  float m_run = -INFINITY, l_run = 0.f;
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  if (warp == kMWarps) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      for (int pg = p_begin; pg < p_end; ++pg) {
        const int it = pg - p_begin, st = it % kMStages;
        if (!mbar_wait(&empty[st], (uint32_t)(((it / kMStages) & 1) ^ 1), dead, status, 970)) break;
        const int page = block_table[b * max_pages + pg];
        uint8_t* dst = smem + st * kMStageBytes;
        mbar_expect_tx(&full[st], kMStageBytes);
        tma_load_2d(dst, &map_k, &full[st], hk * D, page * kTPage);
        tma_load_2d(dst + kMHalf, &map_k, &full[st], hk * D + 64, page * kTPage);
        tma_load_2d(dst + 2 * kMHalf, &map_v, &full[st], hk * D, page * kTPage);
        tma_load_2d(dst + 3 * kMHalf, &map_v, &full[st], hk * D + 64, page * kTPage);
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers
    // Q as the A operand: rows = heads (rows >= G are zero), 8 k-steps of 16 dims
    uint32_t qa[8][2];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = qa[ks][1] = 0u;
      if (grow < G) {
        const __nv_bfloat16* qp = q + (long)b * q_stride + (long)(h0 + grow) * D + ks * 16 + qcol;
        qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
        qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
    }
    const int lm = lane >> 3, lr = lane & 7;      // ldmatrix: this lane addresses row lr of matrix lm
    bool ok = true;
    for (int pg = p_begin + warp; pg < p_end; pg += kMWarps) {
      const int it = pg - p_begin, st = it % kMStages;
      ok = mbar_wait(&full[st], (uint32_t)((it / kMStages) & 1), dead, status, 971);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t sK = smem_u32(smem + st * kMStageBytes);
      const uint32_t sV = sK + 2 * kMHalf;
      // ---- S = Q K^T : two 8-token tiles
      float sc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
        const int tok = nt * 8 + lr;
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {            // two k-steps per ldmatrix.x4
          const int c = kp * 4 + lm;                // 16-byte chunk (8 dims) of the 128-dim row
          const uint32_t addr = sK + (c >> 3) * kMHalf + tok * 128 + (((c & 7) ^ (tok & 7)) << 4);
          uint32_t kb[4];
          ldmatrix_x4(addr, kb);
          mma_bf16_16816(sc[nt], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, kb[0], kb[1]);
          mma_bf16_16816(sc[nt], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, kb[2], kb[3]);
        }
      }
      // ---- online softmax of row `grow` (its 16 scores live in the four lanes of a quad)
      float sv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = pg * kTPage + (j >> 1) * 8 + qcol + (j & 1);
        sv[j] = t < ctx ? sc[j >> 1][j & 1] * scale_log2 : -INFINITY;
      }
      float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float alpha = m_run == -INFINITY ? 0.f : exp2f(m_run - m_new);
      float pv[4], ps = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { pv[j] = m_new == -INFINITY ? 0.f : exp2f(sv[j] - m_new); ps += pv[j]; }
      ps += __shfl_xor_sync(0xffffffffu, ps, 1);
      ps += __shfl_xor_sync(0xffffffffu, ps, 2);
      l_run = l_run * alpha + ps;
      m_run = m_new;
      const uint32_t pa0 = pack_bf16x2(pv[0], pv[1]), pa2 = pack_bf16x2(pv[2], pv[3]);
      // ---- O = alpha * O + P V : sixteen 8-dim tiles, two per ldmatrix.x4.trans
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        o[2 * np][0] *= alpha; o[2 * np][1] *= alpha;
        o[2 * np + 1][0] *= alpha; o[2 * np + 1][1] *= alpha;
        const int tok = (lm & 1) * 8 + lr;
        const int c = np * 2 + (lm >> 1);
        const uint32_t addr = sV + (c >> 3) * kMHalf + tok * 128 + (((c & 7) ^ (tok & 7)) << 4);
        uint32_t vb[4];
        ldmatrix_x4_trans(addr, vb);
        mma_bf16_16816(o[2 * np], pa0, 0u, pa2, 0u, vb[0], vb[1]);
        mma_bf16_16816(o[2 * np + 1], pa0, 0u, pa2, 0u, vb[2], vb[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
    }
    // per-warp state to shared memory: row grow < G; lane holds dims nt*8 + qcol + {0,1}
    if (grow < G) {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        sO[(warp * G + grow) * D + nt * 8 + qcol] = o[nt][0];
        sO[(warp * G + grow) * D + nt * 8 + qcol + 1] = o[nt][1];
      }
      if ((lane & 3) == 0) { sM[grow * kMWarps + warp] = m_run; sL[grow * kMWarps + warp] = l_run; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMWarps; ++w) M = fmaxf(M, sM[g * kMWarps + w]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kMWarps; ++w) {
      const float f = sM[g * kMWarps + w] == -INFINITY ? 0.f : exp2f(sM[g * kMWarps + w] - M);
      L += sL[g * kMWarps + w] * f;
      O += sO[(w * G + g) * D + d] * f;
    }
    if (S == 1) {
      out[(long)b * o_stride + (long)(h0 + g) * D + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
    } else {
      float* pp = part + (((long)b * Hq + h0 + g) * S + sp) * (D + 2);
      pp[d] = O;
      if (d == 0) { pp[D] = M; pp[D + 1] = L; }
    }
  }
}

template <int G>
int launch_mma(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, void* out, float* ws, const int* block_table,
               const int* ctx_lens, dim3 grid, int Hq, int Hkv, int max_pages, float sl2, long q_stride, long o_stride,
               int* status, cudaStream_t stream) {
  const int smem = 1024 + kMStages * kMStageBytes + 2 * kMStages * 8 + 16 + (2 * kMaxG * kMWarps + kMWarps * G * D) * 4;
  auto k = paged_decode_mma_kernel<G>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  k<<<grid, (kMWarps + 1) * 32, smem, stream>>>(mk, mv, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, ws, block_table,
                                                ctx_lens, Hq, Hkv, max_pages, sl2, q_stride, o_stride, status);
  return (int)cudaGetLastError();
}

// One CTA of D threads per (sequence, query head): combines the S partial results.  With `x8`
// given, the result is also written as int8 blocks of 32 with their scales and scaled sums (the
// input format of the decode matrix-vector kernels), one block per warp.
__global__ void __launch_bounds__(D)
paged_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int Hq, int S, long o_stride,
                   int8_t* __restrict__ x8, float* __restrict__ dx, float* __restrict__ sx) {
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const float* pp = part + ((long)b * Hq + h) * S * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < S; ++s) M = fmaxf(M, pp[s * (D + 2) + D]);
  float L = 0.f, O = 0.f;
  for (int s = 0; s < S; ++s) {
    const float ms = pp[s * (D + 2) + D];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
    L += pp[s * (D + 2) + D + 1] * f;
    O += pp[s * (D + 2) + d] * f;
  }
  const __nv_bfloat16 ob = __float2bfloat16(L > 0.f ? O / L : 0.f);
  out[(long)b * o_stride + (long)h * D + d] = ob;
  if (x8 != nullptr) {
    const float v = __bfloat162float(ob);
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax / 127.f;
    const int q = sc > 0.f ? __float2int_rn(v / sc) : 0;
    int qs = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, o);
    const long e = ((long)b * Hq + h) * D + d;
    x8[e] = (int8_t)q;
    if ((d & 31) == 0) { dx[e >> 5] = sc; sx[e >> 5] = sc * (float)qs; }
  }
}

}  // namespace

AX_API int ax_paged_kv_write(const void* k, const void* v, void* kc, void* vc, const int* block_table,
                             const int* seq_ids, const int* positions, int tokens, int Hkv, int Dh,
                             long k_stride, long v_stride, int page_size, int max_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int row = Hkv * Dh;
  if (row % 8 || k_stride % 8 || v_stride % 8) return -1;
  int grid = tokens < 65535 ? tokens : 65535;
  paged_kv_write_kernel<<<grid, 64, 0, stream>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)kc,
                                                 (__nv_bfloat16*)vc, block_table, seq_ids, positions, tokens, row,
                                                 k_stride, v_stride, page_size, max_pages);
  return (int)cudaGetLastError();
}

// q [B, Hq, 128], out [B, Hq, 128] bf16 (row strides in elements); Hq/Hkv in {1, 2, 4, 8}.
// splits > 1 needs `workspace` of B * Hq * splits * 130 floats.  With page_size 16, `num_pages` (pages in the
// cache tensors) and a status word given, the tensor-core kernel runs; otherwise the register-resident one.
AX_API int ax_paged_decode_attention(const void* q, const void* kc, const void* vc, void* out,
                                     const int* block_table, const int* ctx_lens, int B, int Hq, int Hkv,
                                     int Dh, int page_size, int max_pages, float scale, long q_stride,
                                     long o_stride, int splits, float* workspace, int num_pages, int* status,
                                     void* x8, float* dx, float* sx, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (x8 != nullptr && splits < 2) return -3;        // the int8 copy is written by the merge kernel
  if (Dh != D || Hq % Hkv || splits < 1 || (splits > 1 && !workspace)) return -1;
  const int G = Hq / Hkv;
  dim3 grid(B, Hkv, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (page_size == kTPage && num_pages > 0 && status != nullptr) {
    CUtensorMap mk, mv;
    uint64_t dims[2] = {(uint64_t)Hkv * D, (uint64_t)num_pages * page_size};
    uint64_t strides[1] = {(uint64_t)Hkv * D * 2};
    uint32_t box[2] = {64, (uint32_t)kTPage};
    int rc = axh::encode_tensor_map(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kc, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return 1000 + rc;
    rc = axh::encode_tensor_map(&mv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, vc, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return 1100 + rc;
    int e;
    switch (G) {
      case 1: e = launch_mma<1>(mk, mv, q, out, workspace, block_table, ctx_lens, grid, Hq, Hkv, max_pages, sl2, q_stride, o_stride, status, stream); break;
      case 2: e = launch_mma<2>(mk, mv, q, out, workspace, block_table, ctx_lens, grid, Hq, Hkv, max_pages, sl2, q_stride, o_stride, status, stream); break;
      case 4: e = launch_mma<4>(mk, mv, q, out, workspace, block_table, ctx_lens, grid, Hq, Hkv, max_pages, sl2, q_stride, o_stride, status, stream); break;
      case 8: e = launch_mma<8>(mk, mv, q, out, workspace, block_table, ctx_lens, grid, Hq, Hkv, max_pages, sl2, q_stride, o_stride, status, stream); break;
      default: return -2;
    }
    if (e) return e;
    if (splits > 1) {
      paged_merge_kernel<<<dim3(B, Hq), D, 0, stream>>>(workspace, (__nv_bfloat16*)out, Hq, splits, o_stride, (int8_t*)x8, dx, sx);
      return (int)cudaGetLastError();
    }
    return 0;
  }
#define AX_LAUNCH(GG)                                                                                         \
  paged_decode_kernel<GG><<<grid, kWarps * 32, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, \
      (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, workspace, block_table, ctx_lens, Hq, Hkv, page_size,     \
      max_pages, sl2, q_stride, o_stride)
  switch (G) {
    case 1: AX_LAUNCH(1); break;
    case 2: AX_LAUNCH(2); break;
    case 4: AX_LAUNCH(4); break;
    case 8: AX_LAUNCH(8); break;
    default: return -2;
  }
#undef AX_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (splits > 1) {
    paged_merge_kernel<<<dim3(B, Hq), D, 0, stream>>>(workspace, (__nv_bfloat16*)out, Hq, splits, o_stride, (int8_t*)x8, dx, sx);
    e = cudaGetLastError();
  }
  return (int)e;
}
