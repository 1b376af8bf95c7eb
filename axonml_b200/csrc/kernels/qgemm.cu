// Dequantising matmul for decode and small-batch prefill on sm_100a:
//
//     out[b, n] += sum_k x[b, k] * dequant(Wq)[n, k]        (b < 64, Wq in Q4_K or Q8_0)
//
// The weights stay quantised in HBM and are read exactly once.  Per CTA: a tile of 128 weight
// rows x a K-range (split-K over blockIdx.y).  Warp 0 streams the rows' quantised bytes with 1-D
// bulk copies and the activation tile with TMA; warps 2..9 expand 64 weights per row and step to
// bf16 straight into a 128-byte-swizzled shared-memory tile; warp 1 issues tcgen05.mma with the
// WEIGHT tile as the M operand (128 rows) and the batch as the N operand (<= 64), so even batch 1
// runs on the tensor cores; the fp32 accumulator lives in TMEM and is added to `out` with global
// reductions (split-K).
//
// Replaces the reference's "dequantise to f32, then matmul" (crates/axonml-quant/src/dequantize.rs:20-125
// + crates/axonml-nn/src/layers/linear.rs:104-140); Q4_K does not exist there.
#include "common.cuh"

namespace {
using namespace ax;

constexpr int BN = 128;            // weight rows per CTA (MMA M)
constexpr int BB = 64;             // batch columns (MMA N)
constexpr int KS = 256;            // k elements per stage (one Q4_K super-block)
constexpr int kThreads = 320;      // warp 0 TMA, warp 1 MMA, warps 2..9 dequantise (2 threads per row)
constexpr int kATile = BN * 64 * 2;        // 16 KB bf16 tile of one 64-wide step
constexpr int kXStage = 4 * BB * 64 * 2;   // 32 KB: four [64 x 64] slabs of x

template <int QT> struct Q;
template <> struct Q<5> { static constexpr int kRowBytes = 144; static constexpr int kStages = 3; };   // Q4_K
template <> struct Q<0> { static constexpr int kRowBytes = 272; static constexpr int kStages = 2; };   // Q8_0 (8 blocks)

template <int QT>
constexpr int smem_bytes() {
  return 1024 + Q<QT>::kStages * (BN * Q<QT>::kRowBytes + kXStage) + 2 * kATile + 256;
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct QParams {
  const uint8_t* wq;     // row layout: [N][row_bytes]; tiled layout: [N/128][K/256][128][stage row bytes]
  long row_bytes;        // bytes of one full weight row (K/256*144 or K/32*34)
  int tiled;             // 1: the 128 rows of a tile are contiguous per 256-wide k block (one bulk copy)
  float* out;            // [B][N] fp32, accumulated with reductions
  int N, K, B;
  int k_per_split;       // multiple of 256
  int* status;
};

template <int QT>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap map_x, const QParams p) {
  using C = Q<QT>;
  constexpr int kQStage = BN * C::kRowBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sX = smem;                                   // [stages][4 slabs]
  uint8_t* sA = sX + C::kStages * kXStage;              // [2][kATile]
  uint8_t* sQ = sA + 2 * kATile;                        // [stages][BN*row]
  uint64_t* bars = (uint64_t*)(sQ + C::kStages * kQStage);
  uint64_t* full = bars;                  // [stages]
  uint64_t* empty = bars + C::kStages;    // [stages]
  uint64_t* a_full = bars + 2 * C::kStages;      // [2] count 8
  uint64_t* a_free = a_full + 2;                 // [2] count 1 (commit)
  uint64_t* acc_full = a_free + 2;               // 1
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int k_begin = blockIdx.y * p.k_per_split;
  const int k_end = min(p.K, k_begin + p.k_per_split);
  const int nst = (k_end - k_begin + KS - 1) / KS;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < C::kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&a_full[i], 8); mbar_init(&a_free[i], 1); }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<64>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    for (int s = 0; s < nst; ++s) {
      const int st = s % C::kStages;
      const uint32_t ph = (s / C::kStages) & 1;
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(&empty[st], ph ^ 1, dead, p.status, 700);
        if (ok) mbar_expect_tx(&full[st], kQStage + kXStage);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const int k0 = k_begin + s * KS;
      const long koff = (long)(k0 / KS) * C::kRowBytes;
      if (p.tiled) {
        // 128 rows x one k block are contiguous: a single bulk copy instead of 128 small ones
        if (lane == 0)
          bulk_load(sQ + st * kQStage, p.wq + ((long)blockIdx.x * (p.K / KS) + k0 / KS) * kQStage, kQStage, &full[st]);
      } else
#pragma unroll
      for (int i = 0; i < BN / 32; ++i) {
        const int r = i * 32 + lane;
        const int row = min(n0 + r, p.N - 1);          // rows past N re-read the last row (discarded)
        bulk_load(sQ + st * kQStage + r * C::kRowBytes, p.wq + (long)row * p.row_bytes + koff,
                  C::kRowBytes, &full[st]);
      }
      if (lane < 4) tma_load_2d(sX + st * kXStage + lane * (BB * 128), &map_x, &full[st], k0 + lane * 64, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(1, BN, BB, 0, 0);
      int step = 0;
      bool ok = true;
      for (int s = 0; s < nst && ok; ++s) {
        const int st = s % C::kStages;
        const uint32_t ph = (s / C::kStages) & 1;
        ok = mbar_wait(&full[st], ph, dead, p.status, 710);
        for (int sub = 0; sub < 4 && ok; ++sub, ++step) {
          const int ab = step & 1;
          ok = mbar_wait(&a_full[ab], (step >> 1) & 1, dead, p.status, 711);
          if (!ok) break;
          tc_fence_after();
          const uint32_t aA = smem_u32(sA + ab * kATile);
          const uint32_t aX = smem_u32(sX + st * kXStage + sub * (BB * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem, umma_desc_sw128(aA + k * 32, 16, 1024), umma_desc_sw128(aX + k * 32, 16, 1024),
                        idesc, (step | k) != 0);
          umma_commit(&a_free[ab]);
        }
        umma_commit(&empty[st]);
      }
      umma_commit(acc_full);
    }
  } else {
    const int cw = warp - 2;
    const int q = warp & 3;
    const int half = cw >> 2;
    const int r = q * 32 + lane;
    int step = 0;
    bool ok = true;
    for (int s = 0; s < nst && ok; ++s) {
      const int st = s % C::kStages;
      const uint32_t ph = (s / C::kStages) & 1;
      ok = mbar_wait(&full[st], ph, dead, p.status, 720);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint8_t* blk = sQ + st * kQStage + r * C::kRowBytes;
      for (int sub = 0; sub < 4; ++sub, ++step) {
        const int ab = step & 1;
        if (step >= 2) {
          ok = mbar_wait(&a_free[ab], ((step >> 1) - 1) & 1, dead, p.status, 721);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        float w[32];
        if (QT == 5) {
          const float d = __half2float(*reinterpret_cast<const __half*>(blk));
          const float dmin = __half2float(*reinterpret_cast<const __half*>(blk + 2));
          const uint8_t* sc = blk + 4;
          const int j = sub * 2 + half;
          int s6, m6;
          if (j < 4) { s6 = sc[j] & 63; m6 = sc[j + 4] & 63; }
          else { s6 = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
          const float dl = d * s6, ml = dmin * m6;
          const uint4* qs = reinterpret_cast<const uint4*>(blk + 16 + sub * 32);
          const uint4 q0 = qs[0], q1 = qs[1];
          const uint32_t qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t v = half ? (qq[i] >> 4) : qq[i];
#pragma unroll
            for (int b = 0; b < 4; ++b) w[i * 4 + b] = dl * (float)((v >> (8 * b)) & 0xF) - ml;
          }
        } else {
          const uint8_t* b8 = blk + (sub * 2 + half) * 34;
          const float d = __half2float(*reinterpret_cast<const __half*>(b8));
          const unsigned short* qv = reinterpret_cast<const unsigned short*>(b8 + 2);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const unsigned short u = qv[i];
            w[2 * i] = d * (float)(int8_t)(u & 0xff);
            w[2 * i + 1] = d * (float)(int8_t)(u >> 8);
          }
        }
        uint8_t* arow = sA + ab * kATile + r * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 o;
          o.x = pack_bf16x2(w[c * 8 + 0], w[c * 8 + 1]); o.y = pack_bf16x2(w[c * 8 + 2], w[c * 8 + 3]);
          o.z = pack_bf16x2(w[c * 8 + 4], w[c * 8 + 5]); o.w = pack_bf16x2(w[c * 8 + 6], w[c * 8 + 7]);
          *reinterpret_cast<uint4*>(arow + (((half * 4 + c) ^ (r & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[ab]);
      }
    }
    // epilogue: this thread holds row n0+r, batch columns [half*32, half*32+32)
    if (ok) {
      ok = mbar_wait(acc_full, 0, dead, p.status, 722);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && nst > 0) {
      tc_fence_after();
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + half * 32, v);
      tc_wait_ld();
      const int n = n0 + r;
      if (n < p.N) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int b = half * 32 + i;
          if (b < p.B) atomicAdd(p.out + (long)b * p.N + n, __uint_as_float(v[i]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<64>(tmem);
}

template <int QT>
int launch_q(const CUtensorMap& mx, const QParams& p, int splits, cudaStream_t stream) {
  auto k = qgemm_kernel<QT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<QT>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((p.N + BN - 1) / BN, splits);
  k<<<grid, kThreads, smem_bytes<QT>(), stream>>>(mx, p);
  return (int)cudaGetLastError();
}

}  // namespace

// out[B,N] (fp32, must be zeroed or hold a value to accumulate onto) += x[B,K] (bf16) * Wq[N,K]^T.
// tiled = 1: Wq was repacked so that each (128-row tile, 256-wide k block) is contiguous, rows
// padded to a multiple of 128 (see ops/quant.py: tile_weight).
// qtype: 5 = Q4_K, 0 = Q8_0.  K must be a multiple of 256, B <= 64.  `splits` = 0 picks a split-K
// factor that fills the GPU.
AX_API int ax_qgemm(int qtype, const void* wq, const void* x, float* out, int B, int N, int K, int ldx,
                    int splits, int tiled, int* status, cudaStream_t stream) {
  if (B <= 0 || N <= 0 || K <= 0) return 0;
  if (B > BB || K % KS || ldx % 8 || (qtype != 5 && qtype != 0)) return -1;
  CUtensorMap mx;
  uint64_t dims[2] = {(uint64_t)K, (uint64_t)B};
  uint64_t strides[1] = {(uint64_t)ldx * 2};
  uint32_t box[2] = {64, BB};
  int rc = axh::encode_tensor_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box,
                                  CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 1000 + rc;
  const int ntiles = (N + BN - 1) / BN;
  const int kblocks = K / KS;
  if (splits <= 0) {
    splits = (axh::sm_count() + ntiles - 1) / ntiles;
    if (splits > kblocks) splits = kblocks;
    if (splits < 1) splits = 1;
  }
  int per = (kblocks + splits - 1) / splits;
  splits = (kblocks + per - 1) / per;
  QParams p;
  p.wq = (const uint8_t*)wq;
  p.row_bytes = qtype == 5 ? (long)(K / 256) * 144 : (long)(K / 32) * 34;
  p.tiled = tiled;
  p.out = out; p.N = N; p.K = K; p.B = B; p.k_per_split = per * KS; p.status = status;
  return qtype == 5 ? launch_q<5>(mx, p, splits, stream) : launch_q<0>(mx, p, splits, stream);
}
