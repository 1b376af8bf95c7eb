// Dequantising matmul for decode and small-batch prefill on sm_100a:
//
//     out[b, n] += sum_k x[b, k] * dequant(Wq)[n, k]        (b < 64, Wq in Q4_K or Q8_0)
//
// The weights stay quantised in HBM and are read exactly once.  Per CTA: a tile of 128 weight
// rows x a K-range (split-K over blockIdx.y).  Warp 0 streams the rows' quantised bytes with 1-D
// bulk copies and the activation tile with TMA; warps 2..17 expand the weights to
// bf16 straight into a 128-byte-swizzled shared-memory tile; warp 1 issues tcgen05.mma with the
// WEIGHT tile as the M operand (128 rows) and the batch as the N operand (<= 64), so even batch 1
// runs on the tensor cores; the fp32 accumulator lives in TMEM and is added to `out` with global
// reductions (split-K).
//
// The expansion avoids integer-to-float conversions (a quarter-rate pipe that would cap the kernel
// far below HBM speed).  Q4_K: each nibble is placed into the mantissa of the bf16 constant 16.0
// with one byte permute, and one packed bf16 fma per two weights applies scale and minimum
// (w = (16 + q) * d - (16 * d + m)).  Q8_0: each byte goes into the mantissa of 2^23 and the
// packed fp32 add/mul of sm_100 finish it.  Sixteen expander warps (four threads per weight row)
// hand the MMA warp whole chunks of two or four 64-wide slabs, so the per-handshake cost is spread
// over 32..64 weights per thread.  Batches up to 16 use a 16-column MMA and a quarter of the
// activation staging.
//
// Replaces the reference's "dequantise to f32, then matmul" (crates/axonml-quant/src/dequantize.rs:20-125
// + crates/axonml-nn/src/layers/linear.rs:104-140); Q4_K does not exist there.
#include "common.cuh"

namespace {
using namespace ax;

constexpr int BN = 128;            // weight rows per CTA (MMA M)
constexpr int KS = 256;            // k elements per stage (one Q4_K super-block)
constexpr int kComputeWarps = 16;  // four threads per weight row
constexpr int kThreads = (2 + kComputeWarps) * 32;   // warp 0 TMA, warp 1 MMA, then the expanders
constexpr int kATile = BN * 64 * 2;        // 16 KB bf16 slab of one 64-wide step
constexpr int kRing = 2;                   // chunks of expanded weights in flight

template <int QT> struct Q;
template <> struct Q<5> { static constexpr int kRowBytes = 144; };   // Q4_K: one super-block
template <> struct Q<0> { static constexpr int kRowBytes = 272; };   // Q8_0: eight blocks

// Slabs per chunk (the unit handed to the MMA warp): a whole stage for the narrow batch tile, half
// a stage for the wide one, whose activation staging needs the room.
template <int BB> __host__ __device__ constexpr int chunk_slabs() { return BB == 16 ? 4 : 2; }
template <int QT, int BB> __host__ __device__ constexpr int stages() { return QT == 5 ? 3 : 2; }
template <int BB> __host__ __device__ constexpr int x_stage() { return 4 * BB * 128; }      // four [BB x 64] bf16 slabs

template <int QT, int BB>
constexpr int smem_bytes() {
  return 1024 + stages<QT, BB>() * (BN * Q<QT>::kRowBytes + x_stage<BB>()) + kRing * chunk_slabs<BB>() * kATile + 256;
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Explicit shared-space accesses with 32-bit addresses: the base of the dynamic shared memory is
// rounded up by hand, after which the compiler no longer knows the address space and would fall back
// to generic loads (64-bit address arithmetic, long-scoreboard latency).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t a, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// (a.x + s) * m, (a.y + s) * m on the packed fp32 pipe, rounded to a bf16 pair (x in the low half)
__device__ __forceinline__ uint32_t addmul_pack(uint32_t ax, uint32_t ay, float s, float m) {
  uint32_t r;
  asm("{\n\t"
      ".reg .b64 v, t, u;\n\t"
      ".reg .b32 lo, hi;\n\t"
      "mov.b64 v, {%1, %2};\n\t"
      "mov.b64 t, {%3, %3};\n\t"
      "mov.b64 u, {%4, %4};\n\t"
      "add.rn.f32x2 v, v, t;\n\t"
      "mul.rn.f32x2 v, v, u;\n\t"
      "mov.b64 {lo, hi}, v;\n\t"
      "cvt.rn.bf16x2.f32 %0, hi, lo;\n\t"
      "}\n"
      : "=r"(r)
      : "r"(ax), "r"(ay), "f"(s), "f"(m));
  return r;
}
__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
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

// Scale and minimum j (0..7) of a Q4_K super-block as the packed constants of the expansion:
// dl2 = (d * scale) twice, c2 = -(16 * dl + dmin * min) twice, both bf16.
__device__ __forceinline__ void q4k_consts(uint32_t s6, uint32_t m6, float d, float dmin, uint32_t& dl2, uint32_t& c2) {
  const uint32_t dlb = bf16_bits(d * (float)s6);
  const float dl_r = __uint_as_float(dlb << 16);                 // the scale as the fma will see it
  const uint32_t cb = bf16_bits(-(16.f * dl_r + dmin * (float)m6));
  dl2 = dlb | (dlb << 16);
  c2 = cb | (cb << 16);
}

// 32 weights of one row: the HALF of the 64-wide step `sub` of super-block `blk`, expanded into
// four 16-byte chunks of the swizzled A row.
template <int HALF>
__device__ __forceinline__ void expand_q4k(uint32_t blk, int sub, uint32_t dl2, uint32_t c2, uint4* o) {
  const uint4 q0 = lds128(blk + 16 + sub * 32), q1 = lds128(blk + 32 + sub * 32);
  const uint32_t qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // nibble -> bits 3..6 of each byte, bit 7 set: the low byte of bf16 (16 + q)
    const uint32_t t = ((HALF ? (qq[i] >> 1) : (qq[i] << 3)) & 0x78787878u) | 0x80808080u;
    w[2 * i] = fma_bf16x2(prmt(t, 0x41414141u, 0x4140u), dl2, c2);
    w[2 * i + 1] = fma_bf16x2(prmt(t, 0x41414141u, 0x4342u), dl2, c2);
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) o[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}

// Q8_0: block j = sub*2 + HALF of the row's eight 34-byte blocks.  Blocks start on 2-byte
// boundaries, so nine aligned words are fetched and the byte permutes absorb the offset.
template <int HALF>
__device__ __forceinline__ void expand_q80(uint32_t blk, int sub, uint4* o) {
  const uint32_t wp = blk + (sub * 17 + HALF * 8) * 4;
  uint32_t x[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) x[i] = lds32(wp + 4 * i);
  const uint32_t hbits = HALF ? (x[0] >> 16) : (x[0] & 0xffffu);
  const float d = __half2float(__ushort_as_half((unsigned short)hbits));
#pragma unroll
  for (int i = 0; i < 9; ++i) x[i] ^= 0x80808080u;               // int8 -> biased uint8
  constexpr int off = 2 + 2 * HALF;                               // byte of the first weight
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int b = off + 2 * i;
    const uint32_t src = x[b >> 2];
    const uint32_t pos = b & 3;
    const uint32_t f0 = prmt(src, 0x4B000000u, 0x7440u | pos);         // 2^23 + u
    const uint32_t f1 = prmt(src, 0x4B000000u, 0x7440u | (pos + 1));
    w[i] = addmul_pack(f0, f1, -8388736.f, d);                         // (u - 128) * d
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) o[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}

template <int QT, int BB>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap map_x, const QParams p) {
  using C = Q<QT>;
  constexpr int kStages = stages<QT, BB>();
  constexpr int kQStage = BN * C::kRowBytes;
  constexpr int kXStage = x_stage<BB>();
  constexpr int kCols = BB < 32 ? 32 : BB;
  constexpr int CH = chunk_slabs<BB>();          // slabs per chunk
  constexpr int kChunksPerStage = 4 / CH;
  constexpr int kItems = CH / 2;                 // (slab, half) items per thread and chunk
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sX = smem;                                   // [stages][4 slabs]
  uint8_t* sA = sX + kStages * kXStage;                 // [ring][CH][kATile]
  uint8_t* sQ = sA + kRing * CH * kATile;               // [stages][BN*row]
  uint64_t* bars = (uint64_t*)(sQ + kStages * kQStage);
  uint64_t* full = bars;                  // [stages]
  uint64_t* empty = bars + kStages;       // [stages]
  uint64_t* a_full = bars + 2 * kStages;         // [ring] one arrival per expander warp
  uint64_t* a_free = a_full + kRing;             // [ring] count 1 (commit)
  uint64_t* acc_full = a_free + kRing;           // 1
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int k_begin = blockIdx.y * p.k_per_split;
  const int k_end = min(p.K, k_begin + p.k_per_split);
  const int nst = (k_end - k_begin + KS - 1) / KS;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < kRing; ++i) { mbar_init(&a_full[i], kComputeWarps); mbar_init(&a_free[i], 1); }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<kCols>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    int st = 0;
    uint32_t ph = 0;
    for (int s = 0; s < nst; ++s, st = (st + 1 == kStages ? 0 : st + 1), ph ^= (st == 0)) {
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
      } else {
#pragma unroll
        for (int i = 0; i < BN / 32; ++i) {
          const int r = i * 32 + lane;
          const int row = min(n0 + r, p.N - 1);          // rows past N re-read the last row (discarded)
          bulk_load(sQ + st * kQStage + r * C::kRowBytes, p.wq + (long)row * p.row_bytes + koff,
                    C::kRowBytes, &full[st]);
        }
      }
      if (lane < 4) tma_load_2d(sX + st * kXStage + lane * (BB * 128), &map_x, &full[st], k0 + lane * 64, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // One thread feeds the tensor core; its instruction stream is the critical path between
      // "chunk expanded" and "ring slot free", so descriptors are built once and only advanced.
      constexpr uint32_t idesc = umma_idesc_f16(1, BN, BB, 0, 0);
      const uint64_t dA0 = umma_desc_sw128(smem_u32(sA), 16, 1024);
      const uint64_t dX0 = umma_desc_sw128(smem_u32(sX), 16, 1024);
      int st = 0, ring = 0;
      uint32_t ph = 0, rph = 0, acc = 0;
      bool ok = true;
      for (int s = 0; s < nst && ok; ++s) {
        ok = mbar_wait(&full[st], ph, dead, p.status, 710);
#pragma unroll
        for (int c = 0; c < kChunksPerStage; ++c) {
          if (!ok) break;
          ok = mbar_wait(&a_full[ring], rph, dead, p.status, 711);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dA = dA0 + (uint64_t)((ring * CH * kATile) >> 4);
          const uint64_t dX = dX0 + (uint64_t)((st * kXStage + c * CH * (BB * 128)) >> 4);
#pragma unroll
          for (int sl = 0; sl < CH; ++sl) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              umma_f16_ss(tmem, dA + (uint64_t)((sl * kATile + k * 32) >> 4), dX + (uint64_t)((sl * BB * 128 + k * 32) >> 4),
                          idesc, acc);
              acc = 1;
            }
          }
          umma_commit(&a_free[ring]);
          if (++ring == kRing) { ring = 0; rph ^= 1; }
        }
        umma_commit(&empty[st]);
        if (++st == kStages) { st = 0; ph ^= 1; }
      }
      umma_commit(acc_full);
    }
  } else {
    const int cw = warp - 2;
    const int q = warp & 3;                // TMEM lane quarter this warp may read
    const int it = cw >> 2;                // 0..3, warp-uniform: which (slab, half) items of a chunk
    const int half = it & 1;
    const int r = q * 32 + lane;
    const int soff = r & 7;
    const uint32_t sA_u32 = smem_u32(sA);
    int st = 0, ring = 0, ci = 0;
    uint32_t ph = 0, rph = 1;              // rph: parity of the previous use of the ring slot
    int pending = -1;                      // ring slot whose stores still await fence + arrive
    bool ok = true;
    for (int s = 0; s < nst && ok; ++s) {
      ok = mbar_wait(&full[st], ph, dead, p.status, 720);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t blk = smem_u32(sQ) + st * kQStage + r * C::kRowBytes;
      // this thread expands groups `it` and `it + 4` of the eight 32-wide groups of the stage
      uint32_t dl2[2] = {0, 0}, c2[2] = {0, 0};
      if (QT == 5) {
        const uint4 hd = lds128(blk);       // d, dmin and the 12 scale bytes
        const float d = __half2float(__ushort_as_half((unsigned short)(hd.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hd.x >> 16)));
        const uint32_t b0 = (hd.y >> (8 * it)) & 0xffu, b1 = (hd.z >> (8 * it)) & 0xffu, b2 = (hd.w >> (8 * it)) & 0xffu;
        q4k_consts(b0 & 63u, b1 & 63u, d, dmin, dl2[0], c2[0]);                                   // group it
        q4k_consts((b2 & 0xFu) | ((b0 >> 6) << 4), (b2 >> 4) | ((b1 >> 6) << 4), d, dmin, dl2[1], c2[1]);   // it + 4
      }
#pragma unroll
      for (int c = 0; c < kChunksPerStage; ++c, ++ci) {
        uint4 o[kItems][4];
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
          const int sub = c * CH + (it >> 1) + 2 * i;       // 64-wide step of the stage
          const int gi = c * kItems + i;                    // 0: group it, 1: group it + 4
          if (QT == 5) {
            if (half) expand_q4k<1>(blk, sub, dl2[gi], c2[gi], o[i]);
            else expand_q4k<0>(blk, sub, dl2[gi], c2[gi], o[i]);
          } else {
            if (half) expand_q80<1>(blk, sub, o[i]);
            else expand_q80<0>(blk, sub, o[i]);
          }
        }
        // the previous chunk's stores have landed while this one was expanded: publish them now
        if (pending >= 0) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[pending]);
        }
        if (ci >= kRing) {
          ok = mbar_wait(&a_free[ring], rph, dead, p.status, 721);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
          const uint32_t arow = sA_u32 + (ring * CH + (it >> 1) + 2 * i) * kATile + r * 128;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) sts128(arow + (((half * 4 + ch) ^ soff) << 4), o[i][ch]);
        }
        pending = ring;
        if (++ring == kRing) { ring = 0; rph ^= 1; }
      }
      if (++st == kStages) { st = 0; ph ^= 1; }
    }
    if (ok && pending >= 0) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[pending]);
    }
    // epilogue: this thread holds row n0+r; the four warps of a lane quarter split the batch columns
    if (ok) {
      ok = mbar_wait(acc_full, 0, dead, p.status, 722);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && nst > 0 && (BB == 64 || it == 0)) {
      tc_fence_after();
      const int n = n0 + r;
      const int col0 = BB == 64 ? it * 16 : 0;
      uint32_t v[16];
      tmem_ld_32x32b_x16(tmem + ((uint32_t)(q * 32) << 16) + col0, v);
      tc_wait_ld();
      if (n < p.N) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (col0 + i < p.B) atomicAdd(p.out + (long)(col0 + i) * p.N + n, __uint_as_float(v[i]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<kCols>(tmem);
}

template <int QT, int BB>
int launch_q(const void* x, int ldx, QParams p, int splits, cudaStream_t stream) {
  CUtensorMap mx;
  uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.B};
  uint64_t strides[1] = {(uint64_t)ldx * 2};
  uint32_t box[2] = {64, BB};
  int rc = axh::encode_tensor_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box,
                                  CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 1000 + rc;
  auto k = qgemm_kernel<QT, BB>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<QT, BB>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int ntiles = (p.N + BN - 1) / BN;
  const int kblocks = p.K / KS;
  if (splits <= 0) {
    // split-K factor with the fewest (waves x stages per CTA), one stage of fixed cost per CTA
    const int slots = axh::sm_count();
    long best = -1;
    for (int sp = 1; sp <= kblocks && sp <= 64; ++sp) {
      const int per = (kblocks + sp - 1) / sp;
      const int ctas = ntiles * ((kblocks + per - 1) / per);
      const long cost = (long)((ctas + slots - 1) / slots) * (per + 1);
      if (best < 0 || cost < best) { best = cost; splits = sp; }
    }
  }
  const int per = (kblocks + splits - 1) / splits;
  splits = (kblocks + per - 1) / per;
  p.k_per_split = per * KS;
  dim3 grid(ntiles, splits);
  k<<<grid, kThreads, smem_bytes<QT, BB>(), stream>>>(mx, p);
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
  if (B > 64 || K % KS || ldx % 8 || (qtype != 5 && qtype != 0)) return -1;
  QParams p;
  p.wq = (const uint8_t*)wq;
  p.row_bytes = qtype == 5 ? (long)(K / 256) * 144 : (long)(K / 32) * 34;
  p.tiled = tiled;
  p.out = out; p.N = N; p.K = K; p.B = B; p.k_per_split = 0; p.status = status;
  if (B <= 16)
    return qtype == 5 ? launch_q<5, 16>(x, ldx, p, splits, stream) : launch_q<0, 16>(x, ldx, p, splits, stream);
  return qtype == 5 ? launch_q<5, 64>(x, ldx, p, splits, stream) : launch_q<0, 64>(x, ldx, p, splits, stream);
}
