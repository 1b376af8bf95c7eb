// Q4_K matrix-vector products for decode batches of 1..8 rows.
//
// The tensor-core dequantising matmul (qgemm.cu) expands every weight tile through shared memory;
// at batch 1 that work is wasted and the kernel sits at 0.18 of the HBM roofline.  Here a warp
// owns a few consecutive output rows: each lane loads 32 bytes of packed nibbles per row straight
// from global memory (one 64-weight group), splits them into low / high nibbles with two logic ops
// per word and multiplies them against the int8-quantised activations with dp4a (0.5 instructions
// per weight).  The
// activations are quantised once per call into 32-wide blocks (scale and block sum, as llama.cpp's
// Q8_1 does), so that
//     sum_i (d*sc*q_i - dmin*m) * (dx*q8_i) = d*sc*dx * dot(q, q8) - dmin*m * (dx * sum q8).
//
// Weight layouts: GGML row-major super-blocks, or the tile-contiguous layout of qgemm.cu
// ([N/128][K/256][128 rows][144 bytes]).  Super-block: half d, half dmin, 12 bytes of 6-bit
// scales/mins, 128 bytes of nibbles (byte l of group g: low nibble = weight 64g+l, high nibble =
// weight 64g+32+l) - the GGUF Q4_K format the reference's quantiser family extends
// (crates/axonml-quant/src/types.rs:57-67).
#include "common.cuh"

namespace {
using namespace ax;

constexpr int kSB = 144;                   // bytes of one Q4_K super-block (256 weights)

// activations: one warp per 32-wide block
__global__ void __launch_bounds__(256)
q8_quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, long ldx, int8_t* __restrict__ x8, float* __restrict__ dx,
                        float* __restrict__ sx, int B, int K) {
  const int lane = threadIdx.x & 31;
  const long blk = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int per_row = K / 32;
  if (blk >= (long)B * per_row) return;
  const int b = (int)(blk / per_row), i = (int)(blk - (long)b * per_row);
  const float v = __bfloat162float(x[(long)b * ldx + i * 32 + lane]);
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = amax / 127.f;
  const int q = d > 0.f ? __float2int_rn(v / d) : 0;
  int s = q;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  x8[(long)b * K + i * 32 + lane] = (int8_t)q;
  if (lane == 0) { dx[blk] = d; sx[blk] = d * (float)s; }
}

__device__ __forceinline__ void store_out(void* out, int out_bf16, long i, float v) {
  if (out_bf16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16(v);
  else reinterpret_cast<float*>(out)[i] = v;
}

// 6-bit scales and mins of sub-blocks 2g and 2g+1 from the 12 packed bytes (hdr.y, hdr.z, hdr.w):
// bytes 0-3 hold scales 0-3 (low 6 bits) and the top bits of scales 4-7, bytes 4-7 the same for the
// mins, bytes 8-11 the low nibbles of scales / mins 4-7.
__device__ __forceinline__ void scales_of_group(const uint4& hdr, int g, float& sc_lo, float& sc_hi, float& m_lo,
                                                float& m_hi) {
  const int sh = (g & 1) * 16;
  const uint32_t a = (hdr.y >> sh) & 0xffffu, b = (hdr.z >> sh) & 0xffffu, c = (hdr.w >> sh) & 0xffffu;
  uint32_t s0, s1, m0, m1;
  if (g < 2) {
    s0 = a & 63u; s1 = (a >> 8) & 63u;
    m0 = b & 63u; m1 = (b >> 8) & 63u;
  } else {
    s0 = (c & 0xFu) | (((a >> 6) & 3u) << 4);
    s1 = ((c >> 8) & 0xFu) | (((a >> 14) & 3u) << 4);
    m0 = ((c >> 4) & 0xFu) | (((b >> 6) & 3u) << 4);
    m1 = ((c >> 12) & 0xFu) | (((b >> 14) & 3u) << 4);
  }
  sc_lo = (float)s0; sc_hi = (float)s1; m_lo = (float)m0; m_hi = (float)m1;
}

// A lane owns one 64-weight group (32 bytes of nibbles = sub-blocks 2g and 2g+1) of a super-block,
// four lanes a super-block, for R consecutive rows at once: the int8 activations of the group (64
// bytes per batch row) are loaded into registers once and multiplied against R rows, which divides
// the L1 traffic per weight by R (with one row per warp the kernel ran at 86 % of the L1 pipe and
// 2.2 TB/s).
//
// Shapes.  LPR lanes work on one row (LPR / 4 super-blocks per iteration); with short rows (K <
// 2048, tensor-parallel shards) LPR is 16 or 8 and a warp takes 32 / LPR row groups side by side, so
// no lane idles.  With few rows (N of a few thousand) KS warps of a CTA split the super-blocks of
// their rows between them and add their partial sums through shared memory, so that the GPU still
// holds a few thousand warps with loads in flight.
template <int NB, int R, int LPR>
__global__ void __launch_bounds__(256)
q4k_gemv_kernel(const uint8_t* __restrict__ W, const int8_t* __restrict__ x8, const float* __restrict__ dx,
                const float* __restrict__ sx, void* __restrict__ out, int out_bf16, int N, int K, int tiled, int KS) {
  constexpr int SUBS = 32 / LPR;                 // row groups side by side in a warp
  __shared__ float part[8][SUBS * R * NB];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nsb = K / 256, per_row32 = K / 32;
  const int sub = lane / LPR, l = lane % LPR;
  const int sbi = l >> 2, g = l & 3;
  const long sb_stride = tiled ? 128L * kSB : kSB;
  const int ks = warp % KS, wg = warp / KS;      // split index, row-group index inside the CTA
  const int rows_per_cta = (8 / KS) * SUBS * R;
  const int sb_begin = (int)((long)nsb * ks / KS), sb_end = (int)((long)nsb * (ks + 1) / KS);
  for (int base_row = blockIdx.x * rows_per_cta; base_row < N; base_row += gridDim.x * rows_per_cta) {
    const int row0 = base_row + (wg * SUBS + sub) * R;
    const uint8_t* base[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = min(row0 + r, N - 1);                 // rows past the end repeat the last one (not stored)
      base[r] = tiled ? W + ((long)(row >> 7) * nsb) * (128L * kSB) + (long)(row & 127) * kSB : W + (long)row * nsb * kSB;
    }
    float acc[R][NB];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;
    for (int sb0 = sb_begin; sb0 < sb_end; sb0 += LPR / 4) {
      const int sb = sb0 + sbi;
      if (sb < sb_end) {
        const int i32 = sb * 8 + 2 * g;
        const long xo = (long)sb * 256 + g * 64;
        int xl[NB][8], xh[NB][8];
        float2 dd[NB], ss[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int4* xp = reinterpret_cast<const int4*>(x8 + (long)b * K + xo);
          const int4 xa = __ldg(xp), xb = __ldg(xp + 1), xc = __ldg(xp + 2), xd = __ldg(xp + 3);
          xl[b][0] = xa.x; xl[b][1] = xa.y; xl[b][2] = xa.z; xl[b][3] = xa.w;
          xl[b][4] = xb.x; xl[b][5] = xb.y; xl[b][6] = xb.z; xl[b][7] = xb.w;
          xh[b][0] = xc.x; xh[b][1] = xc.y; xh[b][2] = xc.z; xh[b][3] = xc.w;
          xh[b][4] = xd.x; xh[b][5] = xd.y; xh[b][6] = xd.z; xh[b][7] = xd.w;
          dd[b] = __ldg(reinterpret_cast<const float2*>(dx + (long)b * per_row32 + i32));
          ss[b] = __ldg(reinterpret_cast<const float2*>(sx + (long)b * per_row32 + i32));
        }
        uint4 hdr[R], q0[R], q1[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {                         // all weight loads of the R rows in flight together
          const uint8_t* blk = base[r] + sb * sb_stride;
          hdr[r] = __ldg(reinterpret_cast<const uint4*>(blk));
          q0[r] = __ldg(reinterpret_cast<const uint4*>(blk + 16 + g * 32));
          q1[r] = __ldg(reinterpret_cast<const uint4*>(blk + 32 + g * 32));
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const __half2 dm = *reinterpret_cast<const __half2*>(&hdr[r].x);
          const float d = __low2float(dm), dmin = __high2float(dm);
          float sc_lo, sc_hi, m_lo, m_hi;
          scales_of_group(hdr[r], g, sc_lo, sc_hi, m_lo, m_hi);
          const uint32_t qw[8] = {q0[r].x, q0[r].y, q0[r].z, q0[r].w, q1[r].x, q1[r].y, q1[r].z, q1[r].w};
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            int lo = 0, hi = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              lo = __dp4a((int)(qw[k] & 0x0F0F0F0Fu), xl[b][k], lo);
              hi = __dp4a((int)((qw[k] >> 4) & 0x0F0F0F0Fu), xh[b][k], hi);
            }
            acc[r][b] += d * (sc_lo * dd[b].x * (float)lo + sc_hi * dd[b].y * (float)hi) - dmin * (m_lo * ss[b].x + m_hi * ss[b].y);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float v = acc[r][b];
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (KS == 1) {
          if (l == 0 && row0 + r < N) store_out(out, out_bf16, (long)b * N + row0 + r, v);
        } else if (l == 0) {
          part[warp][(sub * R + r) * NB + b] = v;
        }
      }
    if (KS > 1) {                                  // uniform over the CTA: every warp runs the same row loop
      __syncthreads();
      if (ks == 0 && l == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float v = 0.f;
            for (int j = 0; j < KS; ++j) v += part[warp + j][(sub * R + r) * NB + b];
            if (row0 + r < N) store_out(out, out_bf16, (long)b * N + row0 + r, v);
          }
      }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------- Q8_0
// Q8_0 blocks are 34 bytes (half scale + 32 int8), so nothing in a row is 16-byte aligned.  In the
// tile-contiguous layout ([N/128][K/256][128 rows][272 bytes]) the 128 rows of a k block are one
// contiguous 34 KB piece: a producer lane streams the pieces of a row tile through a ring of
// shared-memory stages with bulk copies, and eight warps read them back with 4-byte loads at a
// 68-byte lane stride (17 words: conflict-free).  A lane owns a pair of blocks (68 bytes: word 0 =
// scale 0 + two weights, words 1-7 weights, word 8 = two weights + scale 1, words 9-16 the second
// block), four lanes a row, a warp 16 rows in two passes.
constexpr int kQ8Row = 272;
constexpr int kQ8Stage = 128 * kQ8Row;

__device__ __forceinline__ uint32_t lds32s(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}

__device__ __forceinline__ void bulk_load_g2s(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int NB, int S>
__global__ void __launch_bounds__(288, NB <= 2 ? 2 : 1)
q80_gemv_kernel(const uint8_t* __restrict__ W, const int8_t* __restrict__ x8, const float* __restrict__ dx,
                void* __restrict__ out, int out_bf16, int N, int K, int* status) {
  extern __shared__ uint8_t q8_raw[];
  __shared__ uint64_t full[S], empty[S];
  __shared__ int dead_flag;
  volatile int* dead = &dead_flag;
  const uint32_t stage0 = (smem_u32(q8_raw) + 127u) & ~127u;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nkb = K / 256, per_row32 = K / 32;
  const int tile = blockIdx.x;
  if (threadIdx.x == 0) {
    dead_flag = 0;
    for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 8); }
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 8) {
    if (lane == 0) {
      const uint8_t* src = W + (long)tile * nkb * kQ8Stage;
      for (int i = 0; i < nkb; ++i) {
        const int st = i % S;
        if (i >= S && !mbar_wait(&empty[st], ((i / S) - 1) & 1, dead, status, 760)) break;
        mbar_expect_tx(&full[st], kQ8Stage);
        bulk_load_g2s(stage0 + st * kQ8Stage, src + (long)i * kQ8Stage, kQ8Stage, &full[st]);
      }
    }
    return;
  }
  const int q = lane & 3, rsub = lane >> 2;
  float acc[2][NB];
#pragma unroll
  for (int ps = 0; ps < 2; ++ps)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[ps][b] = 0.f;
  for (int i = 0; i < nkb; ++i) {
    const int st = i % S;
    int xl[NB][8], xh[NB][8];
    float2 dd[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {                       // issued before the wait: independent of the stage
      const int4* xp = reinterpret_cast<const int4*>(x8 + (long)b * K + i * 256 + q * 64);
      const int4 xa = __ldg(xp), xb = __ldg(xp + 1), xc = __ldg(xp + 2), xd = __ldg(xp + 3);
      xl[b][0] = xa.x; xl[b][1] = xa.y; xl[b][2] = xa.z; xl[b][3] = xa.w;
      xl[b][4] = xb.x; xl[b][5] = xb.y; xl[b][6] = xb.z; xl[b][7] = xb.w;
      xh[b][0] = xc.x; xh[b][1] = xc.y; xh[b][2] = xc.z; xh[b][3] = xc.w;
      xh[b][4] = xd.x; xh[b][5] = xd.y; xh[b][6] = xd.z; xh[b][7] = xd.w;
      dd[b] = __ldg(reinterpret_cast<const float2*>(dx + (long)b * per_row32 + i * 8 + 2 * q));
    }
    if (!mbar_wait(&full[st], (i / S) & 1, dead, status, 761)) break;
#pragma unroll
    for (int ps = 0; ps < 2; ++ps) {
      const uint32_t a = stage0 + st * kQ8Stage + (warp * 16 + ps * 8 + rsub) * kQ8Row + q * 68;
      uint32_t w[17];
#pragma unroll
      for (int k = 0; k < 17; ++k) w[k] = lds32s(a + 4 * k);
      const float d0 = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xffffu)));
      const float d1 = __half2float(__ushort_as_half((unsigned short)(w[8] >> 16)));
      uint32_t q0[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) q0[k] = __funnelshift_r(w[k], w[k + 1], 16);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          s0 = __dp4a((int)q0[k], xl[b][k], s0);
          s1 = __dp4a((int)w[9 + k], xh[b][k], s1);
        }
        acc[ps][b] += d0 * dd[b].x * (float)s0 + d1 * dd[b].y * (float)s1;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[st]);
  }
#pragma unroll
  for (int ps = 0; ps < 2; ++ps)
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float v = acc[ps][b];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      const int row = tile * 128 + warp * 16 + ps * 8 + rsub;
      if (q == 0 && row < N) store_out(out, out_bf16, (long)b * N + row, v);
    }
}

}  // namespace

// x [B, K] bf16 (row stride ldx) times Q4_K W[N, K]^T -> out [B, N] (fp32, or bf16 when out_bf16), 1 <= B <= 8,
// K % 256 == 0.
// Scratch (caller-provided): x8 [B*K] int8, dx and sx [B*K/32] fp32.
// `x` may be null: the activations are then already in x8 / dx / sx (written by a producer kernel,
// decode_fused.cu) and no quantiser launch is made.
AX_API int ax_q4k_gemv(const void* W, int tiled, const void* x, long ldx, void* x8, float* dx, float* sx, void* out,
                       int out_bf16, int B, int N, int K, cudaStream_t stream) {
  if (B < 1 || B > 8 || N <= 0 || K <= 0 || K % 256) return -1;
  if ((((uintptr_t)W) | ((uintptr_t)x8)) & 15) return -1;
  if ((((uintptr_t)dx) | ((uintptr_t)sx)) & 7) return -1;
  const long blocks32 = (long)B * (K / 32);
  if (x != nullptr)
    q8_quantize_rows_kernel<<<(int)((blocks32 * 32 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (int8_t*)x8,
                                                                                   dx, sx, B, K);
  // Lanes per row: all 32 unless the row has fewer than 8 super-blocks.  Rows per lane (R): four reuse
  // the activations best.  Then K is split over warps until the GPU holds about 16 warps per SM.
  const int sms = axh::sm_count();
  const int nsb = K / 256;
  const int LPR = nsb >= 5 ? 32 : (nsb >= 3 ? 16 : 8);
  const int SUBS = 32 / LPR;
  int ks_max = 1;                                     // every split keeps at least one full iteration of its lanes
  if (B <= 4)
    while (ks_max < 4 && nsb / (ks_max * 2) >= LPR / 4) ks_max *= 2;
  int R = (B <= 2) ? 4 : 2;
  while (R > 1 && (long)(N / (R * SUBS)) * ks_max < 16L * sms) R /= 2;  // even the widest split would not fill the GPU
  int KS = 1;
  while (KS < ks_max && (long)(N / (R * SUBS)) * KS < 16L * sms) KS *= 2;
  const int rows_per_cta = (8 / KS) * SUBS * R;
  int grid = (N + rows_per_cta - 1) / rows_per_cta;
  const int cap = sms * 8;
  if (grid > cap) grid = cap;
  const auto* w = (const uint8_t*)W;
  const auto* q8 = (const int8_t*)x8;
#define AX_GEMV(NB, RR, LL) q4k_gemv_kernel<NB, RR, LL><<<grid, 256, 0, stream>>>(w, q8, dx, sx, out, out_bf16, N, K, tiled, KS)
#define AX_GEMV_L(NB, RR)                          \
  if (LPR == 32) AX_GEMV(NB, RR, 32);              \
  else if (LPR == 16) AX_GEMV(NB, RR, 16);         \
  else AX_GEMV(NB, RR, 8);
#define AX_GEMV_B(NB)                                             \
  case NB:                                                        \
    if (R == 4 && NB <= 2) { AX_GEMV_L(NB <= 2 ? NB : 1, 4) }     \
    else if (R >= 2) { AX_GEMV_L(NB, 2) }                         \
    else { AX_GEMV_L(NB, 1) }                                     \
    break;
  switch (B) {
    AX_GEMV_B(1) AX_GEMV_B(2) AX_GEMV_B(3) AX_GEMV_B(4) AX_GEMV_B(5) AX_GEMV_B(6) AX_GEMV_B(7) AX_GEMV_B(8)
  }
#undef AX_GEMV_B
#undef AX_GEMV_L
#undef AX_GEMV
  return (int)cudaGetLastError();
}

// The same product for a Q8_0 weight in the tile-contiguous layout (rows padded to a multiple of
// 128), 1 <= B <= 4.  `sx` is scratch of the activation quantiser and not read here.
AX_API int ax_q80_gemv(const void* W, const void* x, long ldx, void* x8, float* dx, float* sx, void* out, int out_bf16, int B,
                       int N, int K, int* status, cudaStream_t stream) {
  if (B < 1 || B > 4 || N <= 0 || K <= 0 || K % 256) return -1;
  if ((((uintptr_t)W) | ((uintptr_t)x8)) & 15) return -1;
  if (((uintptr_t)dx) & 7) return -1;
  const long blocks32 = (long)B * (K / 32);
  if (x != nullptr)      // null: x8 / dx already hold the quantised activations
    q8_quantize_rows_kernel<<<(int)((blocks32 * 32 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (int8_t*)x8,
                                                                                   dx, sx, B, K);
  const int grid = (N + 127) / 128;
  const auto* w = (const uint8_t*)W;
  const auto* q8 = (const int8_t*)x8;
#define AX_GEMV8(NB, S)                                                                                       \
  case NB: {                                                                                                  \
    constexpr int smem = S * kQ8Stage + 128;                                                                  \
    static bool once = false;                                                                                 \
    if (!once) {                                                                                              \
      cudaFuncSetAttribute(q80_gemv_kernel<NB, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);        \
      once = true;                                                                                            \
    }                                                                                                         \
    q80_gemv_kernel<NB, S><<<grid, 288, smem, stream>>>(w, q8, dx, out, out_bf16, N, K, status);             \
  } break;
  switch (B) {
    AX_GEMV8(1, 3) AX_GEMV8(2, 3) AX_GEMV8(3, 5) AX_GEMV8(4, 5)
  }
#undef AX_GEMV8
  return (int)cudaGetLastError();
}
