// Paged KV cache for serving: a write kernel that scatters new K/V rows into cache pages and the
// decode attention kernel (one query token per sequence) that reads K/V through a block table.
//
// Cache layout: k_cache / v_cache [num_pages, page_size, Hkv, D] bf16; block_table [B, max_pages]
// int32; context_lens [B] int32.  Grouped-query attention: the G = Hq/Hkv query heads that share
// a KV head are processed by the same CTA, so each K/V row is read once for all of them.
// One CTA per (sequence, kv head); 4 lanes cooperate on a token (each holds D/4 of the row), so a
// warp covers 8 tokens per iteration with 16-byte loads; every 4-lane group keeps its own online
// softmax state, groups are merged through shared memory at the end.
//
// Replaces the reference's concat-and-grow KVCache (crates/axonml-llm/src/attention.rs:46-70) and
// the full score-matrix attention of crates/axonml-llm/src/llama.rs:429-441 for the decode step.
#include "common.cuh"

namespace {
using namespace ax;

constexpr int kWarps = 4;
constexpr int kGroups = kWarps * 8;     // 4-lane groups per CTA
constexpr int D = 128;
constexpr int kMaxG = 8;                // query heads per KV head handled in one pass

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

template <int G>
__global__ void __launch_bounds__(kWarps * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ block_table, const int* __restrict__ ctx_lens, int Hq, int Hkv,
                    int page_size, int max_pages, float scale_log2, long q_stride, long o_stride) {
  const int b = blockIdx.x, hk = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 3;                      // which quarter of the row this lane holds
  const int grp = warp * 8 + (lane >> 2);        // token slot of this 4-lane group
  const int ctx = ctx_lens[b];
  const int h0 = hk * (Hq / Hkv);
  // query: every lane keeps its 32-element quarter of each of the G heads
  float qv[G][32];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q + (long)b * q_stride + (long)(h0 + g) * D + sub * 32;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 u = *reinterpret_cast<const uint4*>(qp + c * 8);
      const float2 a = unpack_bf16x2(u.x), bb = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), dd = unpack_bf16x2(u.w);
      float* d = &qv[g][c * 8];
      d[0] = a.x; d[1] = a.y; d[2] = bb.x; d[3] = bb.y; d[4] = cc.x; d[5] = cc.y; d[6] = dd.x; d[7] = dd.y;
    }
  }
  float m[G], l[G], acc[G][32];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[g][i] = 0.f;
  }
  const long row = (long)Hkv * D;
  for (int t0 = 0; t0 < ctx; t0 += kGroups) {
    const int t = t0 + grp;
    const bool valid = t < ctx;
    float kf[32], vf[32];
    if (valid) {
      const int page = block_table[b * max_pages + t / page_size];
      const long off = ((long)page * page_size + t % page_size) * row + (long)hk * D + sub * 32;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 uk = *reinterpret_cast<const uint4*>(kc + off + c * 8);
        const uint4 uv = *reinterpret_cast<const uint4*>(vc + off + c * 8);
        float2 a = unpack_bf16x2(uk.x), bb = unpack_bf16x2(uk.y), cc = unpack_bf16x2(uk.z), dd = unpack_bf16x2(uk.w);
        float* d = &kf[c * 8];
        d[0] = a.x; d[1] = a.y; d[2] = bb.x; d[3] = bb.y; d[4] = cc.x; d[5] = cc.y; d[6] = dd.x; d[7] = dd.y;
        a = unpack_bf16x2(uv.x); bb = unpack_bf16x2(uv.y); cc = unpack_bf16x2(uv.z); dd = unpack_bf16x2(uv.w);
        d = &vf[c * 8];
        d[0] = a.x; d[1] = a.y; d[2] = bb.x; d[3] = bb.y; d[4] = cc.x; d[5] = cc.y; d[6] = dd.x; d[7] = dd.y;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
      if (valid) {
#pragma unroll
        for (int i = 0; i < 32; ++i) s += qv[g][i] * kf[i];
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (valid) {
        s *= scale_log2;
        const float mn = fmaxf(m[g], s);
        const float alpha = exp2f(m[g] - mn), pe = exp2f(s - mn);
        l[g] = l[g] * alpha + pe;
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[g][i] = acc[g][i] * alpha + pe * vf[i];
        m[g] = mn;
      }
    }
  }
  // merge the kGroups partial states: shared memory [G][kGroups] for (m, l), then a second pass
  __shared__ float sm[kMaxG][kGroups], sl[kMaxG][kGroups];
  __shared__ float so[kMaxG][D];
  for (int i = threadIdx.x; i < kMaxG * D; i += blockDim.x) (&so[0][0])[i] = 0.f;
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) { sm[g][grp] = m[g]; sl[g][grp] = l[g]; }
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
    for (int j = 0; j < kGroups; ++j) M = fmaxf(M, sm[g][j]);
    float L = 0.f;
    for (int j = 0; j < kGroups; ++j) L += sl[g][j] * (sm[g][j] == -INFINITY ? 0.f : exp2f(sm[g][j] - M));
    const float w = (m[g] == -INFINITY || L <= 0.f) ? 0.f : exp2f(m[g] - M) / L;
#pragma unroll
    for (int i = 0; i < 32; ++i) atomicAdd(&so[g][sub * 32 + i], acc[g][i] * w);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    out[(long)b * o_stride + (long)(h0 + g) * D + d] = __float2bfloat16(so[g][d]);
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
AX_API int ax_paged_decode_attention(const void* q, const void* kc, const void* vc, void* out,
                                     const int* block_table, const int* ctx_lens, int B, int Hq, int Hkv,
                                     int Dh, int page_size, int max_pages, float scale, long q_stride,
                                     long o_stride, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Dh != D || Hq % Hkv) return -1;
  const int G = Hq / Hkv;
  dim3 grid(B, Hkv);
  const float sl2 = scale * 1.4426950408889634f;
#define AX_LAUNCH(GG)                                                                                         \
  paged_decode_kernel<GG><<<grid, kWarps * 32, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, \
      (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, block_table, ctx_lens, Hq, Hkv, page_size, max_pages, sl2, \
      q_stride, o_stride)
  switch (G) {
    case 1: AX_LAUNCH(1); break;
    case 2: AX_LAUNCH(2); break;
    case 4: AX_LAUNCH(4); break;
    default: return -2;
  }
#undef AX_LAUNCH
  return (int)cudaGetLastError();
}
