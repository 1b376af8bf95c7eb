// Implicit-GEMM 2-D convolution (NHWC bf16, fp32 accumulation) on tcgen05:
//
//     y[n, ho, wo, co] = act(bias[co] + sum_{r,s,ci} x[n, sh*ho + r - ph, sw*wo + s - pw, ci] * w[co, r, s, ci])
//
// No im2col matrix is materialised.  A GEMM row is an output pixel; a tile of 128 rows is a
// TN x TH x TW box of pixels, so for filter tap (r, s) and a block of 64 input channels the A
// operand of the tile is simply the same box of the INPUT shifted by (r - ph, s - pw): one 4-D
// tiled TMA load, whose out-of-range coordinates (the zero padding, ragged edges) are filled with
// zeros by the TMA unit.  Shared memory then holds [pixel][64 channels] rows of 128 bytes in the
// 128-byte swizzle: exactly the K-major operand tcgen05.mma wants.  The filter matrix
// [Cout, kh*kw*Cin] is the K-major B operand, loaded as in the plain GEMM.  The K loop runs over
// taps x channel blocks.  The epilogue (bias, optional ReLU) stores each warp's 32 pixels x 64
// channels with one 4-D TMA store, which also clips ragged tiles.
//
// Strides.  For one filter tap the rows sh*ho + r - ph all have the same remainder a modulo sh, so
// they are consecutive rows of the "parity view" a of the input: the tensor map whose base is row a
// and whose row stride is sh rows.  A strided convolution therefore needs sh*sw tensor maps over
// the same memory and a table that gives, per tap, its view and its (dh, dw) shift inside the view;
// the loads stay plain boxes and the out-of-range fill still provides the padding.  The kernel only
// sees the table, so the same code runs
//   * the forward of any stride,
//   * the data gradient of a stride-1 convolution (output gradient as input, filter rotated by 180
//     degrees with its channel dims exchanged, padding k-1-p),
//   * the data gradient of a strided convolution, one launch per parity class (a, b) of the INPUT
//     pixels: dx[sh*i + a, sw*j + b] only receives the taps with r = a + ph (mod sh), s = b + pw (mod sw),
//     a stride-1 problem over dy whose result is stored through a parity view of dx.  No tap is
//     computed that the strided forward did not have (no zero-insertion).
//
// Replaces the reference's 7-deep scalar loop (crates/axonml-nn/src/layers/conv.rs:256-337) and
// its WGSL direct-convolution shader (crates/axonml-core/src/backends/wgpu_backend.rs:1364-1427).
#include "common.cuh"

namespace {
using namespace ax;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
constexpr int kStageBufBytes = 32 * 128;

constexpr int kMaxTaps = 64;

struct XMaps { CUtensorMap m[4]; };     // parity views of the input (one for stride 1)

struct ConvParams {
  int N, Cin, Cout, Ho, Wo;               // Ho, Wo: extents of the output view this launch writes
  int ntaps;
  int8_t tap_map[kMaxTaps], tap_dh[kMaxTaps], tap_dw[kMaxTaps];
  uint8_t tap_wcol[kMaxTaps];             // the tap's column block in the filter matrix [Cout, taps * Cin]
  int TN, TH, TW;          // pixel box of a tile, TN*TH*TW == 128
  int bw, bh, bn;          // pixel box of one epilogue warp, bw*bh*bn == 32
  const void* bias;
  int bias_kind;           // 0 none, 1 fp32, 2 bf16
  int act;
  int* status;
};

template <int BN>
struct Cfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmem = 1024 + kStages * kStage + kEpiWarps * 2 * kStageBufBytes + 256;
};

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int x, int y, int z,
                                             int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               :
               : "l"((uint64_t)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
conv_fprop_kernel(const __grid_constant__ XMaps maps_x, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_y, const __grid_constant__ ConvParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* epi_base = smem + C::kStages * C::kStage;
  uint64_t* bars = (uint64_t*)(epi_base + kEpiWarps * 2 * kStageBufBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* tfull_bar = bars + 2 * C::kStages;
  uint64_t* tempty_bar = bars + 2 * C::kStages + 2;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * C::kStages + 4);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_w = (p.Wo + p.TW - 1) / p.TW;
  const int tiles_h = (p.Ho + p.TH - 1) / p.TH;
  const int tiles_n = (p.N + p.TN - 1) / p.TN;
  const int tiles_c = (p.Cout + BN - 1) / BN;
  const int num_tiles = tiles_w * tiles_h * tiles_n * tiles_c;
  const int cblocks = p.Cin / BK;
  const int num_kb = p.ntaps * cblocks;

  // consecutive tiles share the pixel box (the A operand) and differ in the output-channel block
  auto tile_coords = [&](int t, int& n0, int& h0, int& w0, int& c0) {
    const int cb = t % tiles_c;
    int r = t / tiles_c;
    const int tw = r % tiles_w; r /= tiles_w;
    const int th = r % tiles_h; r /= tiles_h;
    n0 = r * p.TN; h0 = th * p.TH; w0 = tw * p.TW; c0 = cb * BN;
  };

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < C::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], kEpiWarps); }
    mbar_fence_init();
    prefetch_tensormap(&maps_x.m[0]);
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_y);
  }
  if (warp == 1) { tmem_alloc<C::kTmemCols>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int n0, h0, w0, c0;
        tile_coords(t, n0, h0, w0, c0);
        for (int tap = 0; tap < p.ntaps && !*dead; ++tap) {
          const CUtensorMap* mx = &maps_x.m[p.tap_map[tap]];
          const int dh = p.tap_dh[tap], dw = p.tap_dw[tap], wcol = p.tap_wcol[tap] * p.Cin;
          for (int cb = 0; cb < cblocks; ++cb) {
            if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 900)) break;
            uint8_t* sa = stage_base + s * C::kStage;
            mbar_expect_tx(&full_bar[s], C::kStage);
            // the tile's pixel box of the tap's input view, shifted by the tap; padding comes back as zeros
            tma_load_4d(sa, mx, &full_bar[s], cb * BK, w0 + dw, h0 + dh, n0);
            tma_load_2d(sa + C::kStageA, &map_w, &full_bar[s], wcol + cb * BK, c0);
            if (++s == C::kStages) { s = 0; ph ^= 1; }
          }
        }
        if (*dead) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(1, BM, BN, 0, 0);
      // descriptors of stage 0, advanced per stage and k step (keeps the issuing thread short)
      const uint64_t da0 = umma_desc_sw128(smem_u32(stage_base), 16, 1024);
      const uint64_t db0 = umma_desc_sw128(smem_u32(stage_base) + C::kStageA, 16, 1024);
      int s = 0, it = 0;
      uint32_t ph = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, dead, p.status, 910)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, dead, p.status, 911)) break;
          tc_fence_after();
          const uint64_t soff = (uint64_t)((uint32_t)(s * C::kStage) >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_ss(d_tmem, da0 + soff + (uint64_t)(k * ((UMMA_K * 2) >> 4)), db0 + soff + (uint64_t)(k * ((UMMA_K * 2) >> 4)),
                        idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        umma_commit(&tfull_bar[acc]);
        if (*dead) break;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;
    const int ew = warp - 2;
    uint8_t* stg = epi_base + ew * 2 * kStageBufBytes;
    // pixel offset of this warp's 32 rows inside the tile box
    const int idx0 = q * 32;
    const int w_off = idx0 % p.TW, h_off = (idx0 / p.TW) % p.TH, n_off = idx0 / (p.TW * p.TH);
    int buf = 0, it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      int n0, h0, w0, c0;
      tile_coords(t, n0, h0, w0, c0);
      const int acc = it & 1;
      bool ok = mbar_wait(&tfull_bar[acc], (it >> 1) & 1, dead, p.status, 920);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int ch = 0; ch < BN / 64; ++ch) {
        uint32_t r[64];
        {
          uint32_t(&r0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[0]);
          uint32_t(&r1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[32]);
          tmem_ld_32x32b_x32(t_row + ch * 64, r0);
          tmem_ld_32x32b_x32(t_row + ch * 64 + 32, r1);
          tc_wait_ld();
        }
        if (ch == BN / 64 - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        }
        const int co0 = c0 + ch * 64;
        if (co0 >= p.Cout) continue;
        add_bias_chunk(r, p.bias, p.bias_kind, co0, p.Cout);
        apply_act_chunk(r, p.act);
        uint8_t* dst = stg + buf * kStageBufBytes;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[c * 8 + 0]), __uint_as_float(r[c * 8 + 1]));
          o.y = pack_bf16x2(__uint_as_float(r[c * 8 + 2]), __uint_as_float(r[c * 8 + 3]));
          o.z = pack_bf16x2(__uint_as_float(r[c * 8 + 4]), __uint_as_float(r[c * 8 + 5]));
          o.w = pack_bf16x2(__uint_as_float(r[c * 8 + 6]), __uint_as_float(r[c * 8 + 7]));
          *reinterpret_cast<uint4*>(dst + lane * 128 + ((c ^ (lane & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();
        __syncwarp();
        // a warp box that starts outside the output (ragged tile) is skipped: TMA stores must not
        // start at an out-of-range coordinate; boxes that start inside are clipped by the unit
        if (lane == 0 && w0 + w_off < p.Wo && h0 + h_off < p.Ho && n0 + n_off < p.N) {
          tma_store_4d(&map_y, dst, co0, w0 + w_off, h0 + h_off, n0 + n_off);
          tma_store_commit();
        }
        buf ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<C::kTmemCols>(tmem_base);
}

template <int BN>
int launch(const XMaps& mx, const CUtensorMap& mw, const CUtensorMap& my, const ConvParams& p, int max_ctas,
           cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = conv_fprop_kernel<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const long tiles = (long)((p.Wo + p.TW - 1) / p.TW) * ((p.Ho + p.TH - 1) / p.TH) * ((p.N + p.TN - 1) / p.TN) *
                     ((p.Cout + BN - 1) / BN);
  int grid = tiles < max_ctas ? (int)tiles : max_ctas;
  if (grid < 1) grid = 1;
  kern<<<grid, kThreads, C::kSmem, stream>>>(mx, mw, my, p);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ weight gradient
//   dw[co, r, s, ci] = sum_{n, ho, wo} dy[n, ho, wo, co] * x[n, sh*ho + r - ph, sw*wo + s - pw, ci]
// as a GEMM whose reduction dimension is the pixels: for one filter tap, M = 128 output channels,
// N = BNC input channels, K = boxes of 64 pixels.  Both operands are "MN-major" (the channel is the
// contiguous dimension in memory): the A slabs are 4-D TMA boxes of dy, the B slabs the same pixel
// box of the tap's parity view of x, shifted by the tap (zero fill = padding).  The pixel range is
// split over CTAs; partial sums are added to an fp32 buffer with global reductions.
constexpr int WBK = 64;          // pixels per k block

struct WgradParams {
  int N, H, W, Cin, Cout, Ho, Wo;
  int kh, kw, ph, pw, sh, sw;
  int TN, TH, TW;          // pixel box of a k block, TN*TH*TW == 64
  int splits;              // pixel-range splits per (tap, co block, ci block)
  float* dw;               // [Cout, kh, kw, Cin] fp32, zero-initialised by the caller
  int* status;
};

template <int BNC>
struct WCfg {
  static constexpr int kStageA = 2 * WBK * 128;             // two 64-channel slabs of dy
  static constexpr int kStageB = (BNC / 64) * WBK * 128;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = BNC == 128 ? 6 : 8;
  static constexpr int kSmem = 1024 + kStages * kStage + 256;
};

template <int BNC>
__global__ void __launch_bounds__(kThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ XMaps maps_x,
                  const WgradParams p) {
  using C = WCfg<BNC>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint64_t* bars = (uint64_t*)(smem + C::kStages * C::kStage);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* tfull_bar = bars + 2 * C::kStages;       // accumulator complete
  uint64_t* tempty_bar = tfull_bar + 1;              // accumulator drained by the epilogue
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 1);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_w = (p.Wo + p.TW - 1) / p.TW, tiles_h = (p.Ho + p.TH - 1) / p.TH, tiles_n = (p.N + p.TN - 1) / p.TN;
  const int nboxes = tiles_w * tiles_h * tiles_n;
  const int co_blocks = (p.Cout + 127) / 128, ci_blocks = p.Cin / BNC;
  const int taps = p.kh * p.kw;
  const int items = taps * co_blocks * ci_blocks * p.splits;
  const int per_split = (nboxes + p.splits - 1) / p.splits;

  auto item_coords = [&](int it, int& tap, int& cob, int& cib, int& b0, int& b1) {
    const int sp = it % p.splits; it /= p.splits;
    cib = it % ci_blocks; it /= ci_blocks;
    cob = it % co_blocks; it /= co_blocks;
    tap = it;
    b0 = sp * per_split;
    b1 = min(nboxes, b0 + per_split);
  };

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < C::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, kEpiWarps);
    mbar_fence_init();
    prefetch_tensormap(&map_dy);
    prefetch_tensormap(&maps_x.m[0]);
  }
  if (warp == 1) { tmem_alloc<BNC>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = blockIdx.x; it < items && !*dead; it += gridDim.x) {
        int tap, cob, cib, b0, b1;
        item_coords(it, tap, cob, cib, b0, b1);
        const int r = tap / p.kw, sx = tap % p.kw;
        // view and shift of this tap: sh*ho + r - ph = sh*(ho + dh) + a with 0 <= a < sh
        const int a = (((r - p.ph) % p.sh) + p.sh) % p.sh, dh = (r - p.ph - a) / p.sh;
        const int bb = (((sx - p.pw) % p.sw) + p.sw) % p.sw, dw = (sx - p.pw - bb) / p.sw;
        const CUtensorMap* mx = &maps_x.m[a * p.sw + bb];
        for (int b = b0; b < b1; ++b) {
          const int tw = b % tiles_w, th = (b / tiles_w) % tiles_h, tn = b / (tiles_w * tiles_h);
          const int w0 = tw * p.TW, h0 = th * p.TH, n0 = tn * p.TN;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 930)) break;
          uint8_t* sa = stage_base + s * C::kStage;
          mbar_expect_tx(&full_bar[s], C::kStage);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tma_load_4d(sa + j * (WBK * 128), &map_dy, &full_bar[s], cob * 128 + j * 64, w0, h0, n0);
#pragma unroll
          for (int j = 0; j < BNC / 64; ++j)
            tma_load_4d(sa + C::kStageA + j * (WBK * 128), mx, &full_bar[s], cib * BNC + j * 64, w0 + dw, h0 + dh, n0);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(1, 128, BNC, 1, 1);
      int s = 0, n_it = 0;
      uint32_t ph = 0;
      for (int it = blockIdx.x; it < items; it += gridDim.x, ++n_it) {
        int tap, cob, cib, b0, b1;
        item_coords(it, tap, cob, cib, b0, b1);
        if (!mbar_wait(tempty_bar, (n_it & 1) ^ 1, dead, p.status, 940)) break;
        tc_fence_after();
        for (int b = b0; b < b1; ++b) {
          if (!mbar_wait(&full_bar[s], ph, dead, p.status, 941)) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * C::kStage);
          const uint32_t sb = sa + C::kStageA;
#pragma unroll
          for (int k = 0; k < WBK / UMMA_K; ++k)
            umma_f16_ss(tmem_base, umma_desc_sw128(sa + k * (UMMA_K * 128), WBK * 128, 1024),
                        umma_desc_sw128(sb + k * (UMMA_K * 128), WBK * 128, 1024), idesc, (b > b0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        umma_commit(tfull_bar);
        if (*dead) break;
      }
    }
  } else {
    const int q = warp & 3;
    int n_it = 0;
    const long row_stride = (long)p.kh * p.kw * p.Cin;
    for (int it = blockIdx.x; it < items; it += gridDim.x, ++n_it) {
      int tap, cob, cib, b0, b1;
      item_coords(it, tap, cob, cib, b0, b1);
      bool ok = mbar_wait(tfull_bar, n_it & 1, dead, p.status, 950);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int co = cob * 128 + q * 32 + lane;
      float* drow = p.dw + (long)co * row_stride + (long)tap * p.Cin + cib * BNC;
#pragma unroll 1
      for (int ch = 0; ch < BNC / 32; ++ch) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + ch * 32, v);
        tc_wait_ld();
        if (b1 > b0 && co < p.Cout) {
#pragma unroll
          for (int j = 0; j < 32; ++j) atomicAdd(drow + ch * 32 + j, __uint_as_float(v[j]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<BNC>(tmem_base);
}

template <int BNC>
int launch_wgrad(const CUtensorMap& mdy, const XMaps& mx, const WgradParams& p, int grid, cudaStream_t stream) {
  using C = WCfg<BNC>;
  auto kern = conv_wgrad_kernel<BNC>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, kThreads, C::kSmem, stream>>>(mdy, mx, p);
  return (int)cudaGetLastError();
}

}  // namespace

namespace {

// floor division and the matching non-negative remainder
inline int floordiv(int a, int b) { int q = a / b; return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q; }

// Tensor maps of the sh*sw parity views of an NHWC tensor: view (a, b) holds the pixels
// (sh*i + a, sw*j + b).  valid[a*sw+b] is 0 for a view without pixels.
int encode_parity_views(XMaps* out, int* valid, const void* x, int N, int H, int W, int C, int sh, int sw,
                        const uint32_t box[4]) {
  for (int a = 0; a < sh; ++a)
    for (int b = 0; b < sw; ++b) {
      const int Ha = (H - a + sh - 1) / sh, Wb = (W - b + sw - 1) / sw;
      valid[a * sw + b] = Ha > 0 && Wb > 0;
      if (!valid[a * sw + b]) continue;
      const uint8_t* base = (const uint8_t*)x + ((long)a * W + b) * C * 2;
      uint64_t dims[4] = {(uint64_t)C, (uint64_t)Wb, (uint64_t)Ha, (uint64_t)N};
      uint64_t strides[3] = {(uint64_t)sw * C * 2, (uint64_t)sh * W * C * 2, (uint64_t)H * W * C * 2};
      int rc = axh::encode_tensor_map(&out->m[a * sw + b], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides,
                                      box, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
    }
  return 0;
}

struct TapList { int n = 0; int map[kMaxTaps], dh[kMaxTaps], dw[kMaxTaps], wcol[kMaxTaps]; };

// One launch of the tap-table kernel.  The input x [N, H, W, Cin] is read through its xsh*xsw parity
// views; the filter matrix is w [Cout, wtaps * Cin]; the output view has extents [N, Ho, Wo, Cout],
// starts y_off elements into y and has the given element strides between columns, rows and images.
int run_taps(const void* x, int N, int H, int W, int Cin, int xsh, int xsw, const TapList& taps, const void* w,
             int wtaps, void* y, int Ho, int Wo, int Cout, long y_off, long y_sw, long y_sh, long y_sn,
             const void* bias, int bias_kind, int act, int max_ctas, int* status, cudaStream_t stream) {
  if (N <= 0 || Ho <= 0 || Wo <= 0) return 0;
  if (Cin % 64 || Cout % 64 || taps.n < 1 || taps.n > kMaxTaps || xsh * xsw > 4 || wtaps > 255) return -1;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return -1;
  if ((y_off | y_sw | y_sh | y_sn) % 8) return -1;
  int sms = axh::sm_count();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;

  // pixel box of a tile: the TW x TH x TN split of 128 that wastes the fewest rows on ragged edges
  int TW = 1, TH = 1, TN = 128;
  double best = -1.0;
  for (int tw = 1; tw <= 128; tw *= 2)
    for (int th = 1; tw * th <= 128; th *= 2) {
      const int tn = 128 / (tw * th);
      const double eff = (double)Wo / (((Wo + tw - 1) / tw) * tw) * ((double)Ho / (((Ho + th - 1) / th) * th)) *
                         ((double)N / (((N + tn - 1) / tn) * tn));
      if (eff > best + 1e-9 || (eff > best - 1e-9 && tw > TW)) { best = eff; TW = tw; TH = th; TN = tn; }
    }
  ConvParams p;
  memset(&p, 0, sizeof(p));
  p.N = N; p.Cin = Cin; p.Cout = Cout; p.Ho = Ho; p.Wo = Wo;
  p.TN = TN; p.TH = TH; p.TW = TW;
  // the 32 pixels of one epilogue warp, in (n, h, w) order with w fastest
  if (TW >= 32) { p.bw = 32; p.bh = 1; p.bn = 1; }
  else if (TW * TH >= 32) { p.bw = TW; p.bh = 32 / TW; p.bn = 1; }
  else { p.bw = TW; p.bh = TH; p.bn = 32 / (TW * TH); }
  p.bias = bias; p.bias_kind = bias ? bias_kind : 0; p.act = act; p.status = status;

  int BN = Cout % 256 == 0 ? 256 : (Cout % 128 == 0 ? 128 : 64);
  // small problems: prefer more tiles over wide tiles
  {
    const long pix_tiles = (long)((Wo + TW - 1) / TW) * ((Ho + TH - 1) / TH) * ((N + TN - 1) / TN);
    while (BN > 64 && pix_tiles * (Cout / BN) < max_ctas) BN /= 2;
  }

  XMaps mx;
  CUtensorMap mw, my;
  int valid[4] = {0, 0, 0, 0};
  {
    uint32_t box[4] = {64, (uint32_t)TW, (uint32_t)TH, (uint32_t)TN};
    int rc = encode_parity_views(&mx, valid, x, N, H, W, Cin, xsh, xsw, box);
    if (rc) return 1000 + rc;
  }
  // taps whose view has no pixels read nothing but padding
  for (int t = 0; t < taps.n; ++t) {
    if (taps.map[t] < 0 || taps.map[t] >= xsh * xsw || !valid[taps.map[t]]) continue;
    if (taps.dh[t] < -128 || taps.dh[t] > 127 || taps.dw[t] < -128 || taps.dw[t] > 127) return -1;
    p.tap_map[p.ntaps] = (int8_t)taps.map[t];
    p.tap_dh[p.ntaps] = (int8_t)taps.dh[t];
    p.tap_dw[p.ntaps] = (int8_t)taps.dw[t];
    p.tap_wcol[p.ntaps] = (uint8_t)taps.wcol[t];
    ++p.ntaps;
  }
  if (p.ntaps == 0) return -1;
  {
    uint64_t dims[2] = {(uint64_t)wtaps * Cin, (uint64_t)Cout};
    uint64_t strides[1] = {(uint64_t)wtaps * Cin * 2};
    uint32_t box[2] = {64, (uint32_t)BN};
    int rc = axh::encode_tensor_map(&mw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return 2000 + rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)Cout, (uint64_t)Wo, (uint64_t)Ho, (uint64_t)N};
    uint64_t strides[3] = {(uint64_t)y_sw * 2, (uint64_t)y_sh * 2, (uint64_t)y_sn * 2};
    uint32_t box[4] = {64, (uint32_t)p.bw, (uint32_t)p.bh, (uint32_t)p.bn};
    int rc = axh::encode_tensor_map(&my, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, (uint8_t*)y + y_off * 2, dims, strides,
                                    box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return 3000 + rc;
  }
  switch (BN) {
    case 256: return launch<256>(mx, mw, my, p, max_ctas, stream);
    case 128: return launch<128>(mx, mw, my, p, max_ctas, stream);
    default: return launch<64>(mx, mw, my, p, max_ctas, stream);
  }
}

}  // namespace

// x [N, H, W, Cin] bf16 (NHWC), w [Cout, kh, kw, Cin] bf16, y [N, Ho, Wo, Cout] bf16 with
// Ho = (H + 2*ph - kh) / sh + 1, Wo = (W + 2*pw - kw) / sw + 1.  Cin and Cout multiples of 64,
// sh * sw <= 4, kh * kw <= 64.  Returns a cudaError_t value, -1 for an unsupported argument.
AX_API int ax_conv2d_fprop(const void* x, const void* w, void* y, const void* bias, int bias_kind, int act, int N,
                           int H, int W, int Cin, int Cout, int kh, int kw, int ph, int pw, int sh, int sw,
                           int max_ctas, int* status, cudaStream_t stream) {
  if (kh < 1 || kw < 1 || sh < 1 || sw < 1 || kh * kw > kMaxTaps) return -1;
  if (H + 2 * ph < kh || W + 2 * pw < kw) return 0;
  const int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  TapList taps;
  for (int r = 0; r < kh; ++r)
    for (int s = 0; s < kw; ++s) {
      const int dh = floordiv(r - ph, sh), dw = floordiv(s - pw, sw);
      const int a = r - ph - dh * sh, b = s - pw - dw * sw;
      taps.map[taps.n] = a * sw + b; taps.dh[taps.n] = dh; taps.dw[taps.n] = dw; taps.wcol[taps.n] = r * kw + s;
      ++taps.n;
    }
  return run_taps(x, N, H, W, Cin, sh, sw, taps, w, kh * kw, y, Ho, Wo, Cout, 0, Cout, (long)Wo * Cout,
                  (long)Ho * Wo * Cout, bias, bias_kind, act, max_ctas, status, stream);
}

// One parity class (a, b) of the data gradient of a strided convolution: the pixels
// dx[n, sh*i + a, sw*j + b, :] of dx [N, H, W, Cin] from dy [N, Ho, Wo, Cout] and the class's filter
// matrix wc [Cin, ntaps * Cout] (tap t of the class: filter position (r_t, s_t), listed by the caller
// as the shifts dh[t] = (a + ph - r_t) / sh, dw[t] = (b + pw - s_t) / sw).
AX_API int ax_conv2d_dgrad_class(const void* dy, const void* wc, void* dx, int N, int H, int W, int Cin, int Ho,
                                 int Wo, int Cout, int sh, int sw, int a, int b, int ntaps, const int* dh,
                                 const int* dw, int max_ctas, int* status, cudaStream_t stream) {
  if (ntaps < 1 || ntaps > kMaxTaps || a < 0 || a >= sh || b < 0 || b >= sw) return -1;
  const int Ha = (H - a + sh - 1) / sh, Wb = (W - b + sw - 1) / sw;
  if (Ha <= 0 || Wb <= 0) return 0;
  TapList taps;
  for (int t = 0; t < ntaps; ++t) {
    taps.map[t] = 0; taps.dh[t] = dh[t]; taps.dw[t] = dw[t]; taps.wcol[t] = t;
  }
  taps.n = ntaps;
  return run_taps(dy, N, Ho, Wo, Cout, 1, 1, taps, wc, ntaps, dx, Ha, Wb, Cin, ((long)a * W + b) * Cin,
                  (long)sw * Cin, (long)sh * W * Cin, (long)H * W * Cin, nullptr, 0, 0, max_ctas, status, stream);
}

// dy [N, Ho, Wo, Cout] bf16, x [N, H, W, Cin] bf16 (NHWC), dw [Cout, kh, kw, Cin] fp32 which must be
// zero on entry (partial sums are added).  Cin and Cout multiples of 64, sh * sw <= 4; every parity
// view of x must hold at least one pixel (H >= sh, W >= sw).
AX_API int ax_conv2d_wgrad(const void* dy, const void* x, float* dw, int N, int H, int W, int Cin, int Cout, int kh,
                           int kw, int ph, int pw, int sh, int sw, int max_ctas, int* status, cudaStream_t stream) {
  if (sh < 1 || sw < 1 || sh * sw > 4 || H < sh || W < sw || kh < 1 || kw < 1) return -1;
  if (H + 2 * ph < kh || W + 2 * pw < kw) return 0;
  const int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  if (N <= 0 || Ho <= 0 || Wo <= 0) return 0;
  if (Cin % 64 || Cout % 64) return -1;
  if (((uintptr_t)dy | (uintptr_t)x | (uintptr_t)dw) & 15) return -1;
  int sms = axh::sm_count();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;
  int TW = 1, TH = 1, TN = 64;
  double best = -1.0;
  for (int tw = 1; tw <= 64; tw *= 2)
    for (int th = 1; tw * th <= 64; th *= 2) {
      const int tn = 64 / (tw * th);
      const double eff = (double)Wo / (((Wo + tw - 1) / tw) * tw) * ((double)Ho / (((Ho + th - 1) / th) * th)) *
                         ((double)N / (((N + tn - 1) / tn) * tn));
      if (eff > best + 1e-9 || (eff > best - 1e-9 && tw > TW)) { best = eff; TW = tw; TH = th; TN = tn; }
    }
  const int BNC = Cin % 128 == 0 ? 128 : 64;
  WgradParams p;
  p.N = N; p.H = H; p.W = W; p.Cin = Cin; p.Cout = Cout; p.Ho = Ho; p.Wo = Wo;
  p.kh = kh; p.kw = kw; p.ph = ph; p.pw = pw; p.sh = sh; p.sw = sw; p.TN = TN; p.TH = TH; p.TW = TW;
  p.dw = dw; p.status = status;
  const int nboxes = ((Wo + TW - 1) / TW) * ((Ho + TH - 1) / TH) * ((N + TN - 1) / TN);
  const int base_items = kh * kw * ((Cout + 127) / 128) * (Cin / BNC);
  int splits = (2 * max_ctas + base_items - 1) / base_items;
  if (splits > nboxes) splits = nboxes;
  if (splits < 1) splits = 1;
  p.splits = splits;
  const long items = (long)base_items * splits;
  const int grid = items < max_ctas ? (int)items : max_ctas;
  CUtensorMap mdy;
  XMaps mx;
  {
    uint64_t dims[4] = {(uint64_t)Cout, (uint64_t)Wo, (uint64_t)Ho, (uint64_t)N};
    uint64_t strides[3] = {(uint64_t)Cout * 2, (uint64_t)Wo * Cout * 2, (uint64_t)Ho * Wo * Cout * 2};
    uint32_t box[4] = {64, (uint32_t)TW, (uint32_t)TH, (uint32_t)TN};
    int rc = axh::encode_tensor_map(&mdy, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dy, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return 1000 + rc;
  }
  {
    uint32_t box[4] = {64, (uint32_t)TW, (uint32_t)TH, (uint32_t)TN};
    int valid[4];
    int rc = encode_parity_views(&mx, valid, x, N, H, W, Cin, sh, sw, box);
    if (rc) return 2000 + rc;
  }
  return BNC == 128 ? launch_wgrad<128>(mdy, mx, p, grid, stream) : launch_wgrad<64>(mdy, mx, p, grid, stream);
}

// ---------------------------------------------------------------------------- im2col for thin inputs
// Convolutions whose input has fewer than 64 channels (an RGB stem) cannot use the tap-wise TMA
// path (its boxes are 64 channels wide).  Their patches are gathered into a matrix col[N*Ho*Wo, Kp]
// which the tcgen05 GEMM multiplies by the [Cout, Kp] filter matrix; the product is the NHWC output.
// One filter row of a patch is KW*C contiguous input values; it is stored padded to RP (a multiple
// of 8) values, k = kh*RP + kw*C + c, so every 16-byte chunk of `col` comes from one contiguous run
// of the input and no index needs a division by C.  Columns past KH*RP are zero.
namespace {
__global__ void __launch_bounds__(256)
im2col_nhwc_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col, int Nimg, int H, int W, int C,
                   int Ho, int Wo, int KH, int KW, int stride, int pad_h, int pad_w, int RP, int Kp) {
  const int cpr = RP / 8;                     // chunks per filter row
  const int chunks = Kp / 8;                  // chunks per output pixel
  const long total = (long)Nimg * Ho * Wo * chunks;
  const int row_run = KW * C;
  const __nv_bfloat16 zero = __float2bfloat16(0.f);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int cc = (int)(i % chunks);
    long r = i / chunks;
    const int wo = (int)(r % Wo); r /= Wo;
    const int ho = (int)(r % Ho);
    const int n = (int)(r / Ho);
    const int kh = cc / cpr, c8 = cc - kh * cpr;
    const int h = ho * stride - pad_h + kh;
    const int w0 = wo * stride - pad_w;
    __nv_bfloat16 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = zero;
    if (kh < KH && h >= 0 && h < H) {
      const __nv_bfloat16* src = x + (((long)n * H + h) * W + w0) * C;     // run start (may lie left of the row)
      const int lo = -w0 * C, hi = (W - w0) * C;                           // valid offsets inside the image row
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = c8 * 8 + j;
        if (t < row_run && t >= lo && t < hi) v[j] = src[t];
      }
    }
    *reinterpret_cast<uint4*>(col + i * 8) = *reinterpret_cast<const uint4*>(v);
  }
}
// Same result, one CTA per output row (n, ho): the KH input rows the row needs are brought into
// shared memory with 16-byte loads (rows outside the image as zeros), and every 16-byte chunk of
// `col` is assembled from shared memory.  Needs W*C % 8 == 0 (16-byte rows) and KH rows to fit.
__global__ void __launch_bounds__(256)
im2col_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col, int H, int W, int C, int Ho,
                   int Wo, int KH, int KW, int stride, int pad_h, int pad_w, int RP, int Kp) {
  extern __shared__ __align__(16) __nv_bfloat16 rows[];          // [KH][W*C]
  const int n = blockIdx.x / Ho, ho = blockIdx.x - n * Ho;
  const int rowlen = W * C, vec_per_row = rowlen / 8;
  for (int i = threadIdx.x; i < KH * vec_per_row; i += blockDim.x) {
    const int kh = i / vec_per_row, v = i - kh * vec_per_row;
    const int h = ho * stride - pad_h + kh;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (h >= 0 && h < H) val = *reinterpret_cast<const uint4*>(x + ((long)n * H + h) * rowlen + v * 8);
    *reinterpret_cast<uint4*>(rows + kh * rowlen + v * 8) = val;
  }
  __syncthreads();
  const int cpr = RP / 8, chunks = Kp / 8, row_run = KW * C;
  const __nv_bfloat16 zero = __float2bfloat16(0.f);
  __nv_bfloat16* out = col + ((long)n * Ho + ho) * Wo * Kp;
  for (int i = threadIdx.x; i < Wo * chunks; i += blockDim.x) {
    const int wo = i / chunks, cc = i - wo * chunks;
    const int kh = cc / cpr, c8 = cc - kh * cpr;
    __nv_bfloat16 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = zero;
    if (kh < KH) {
      const int start = (wo * stride - pad_w) * C;                 // offset of the run inside the image row
      const __nv_bfloat16* src = rows + kh * rowlen;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = c8 * 8 + j, o = start + t;
        if (t < row_run && o >= 0 && o < rowlen) v[j] = src[o];
      }
    }
    *reinterpret_cast<uint4*>(out + (long)i * 8) = *reinterpret_cast<const uint4*>(v);
  }
}
}  // namespace

// x: NHWC bf16 [N, H, W, C]; col: [N*Ho*Wo, Kp] bf16; RP = KW*C rounded up to a multiple of 8,
// Kp a multiple of 8 with Kp >= KH*RP.
AX_API int ax_im2col_nhwc(const void* x, void* col, int N, int H, int W, int C, int KH, int KW, int stride, int pad_h,
                          int pad_w, int RP, int Kp, cudaStream_t stream) {
  if (N <= 0 || C <= 0 || KH <= 0 || KW <= 0 || stride <= 0 || RP % 8 || RP < KW * C || Kp % 8 || Kp < KH * RP) return -1;
  const int Ho = (H + 2 * pad_h - KH) / stride + 1, Wo = (W + 2 * pad_w - KW) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return -1;
  const size_t row_smem = (size_t)KH * W * C * sizeof(__nv_bfloat16);
  if ((W * C) % 8 == 0 && row_smem <= 48 * 1024 && (((uintptr_t)x) & 15) == 0 && Wo * (Kp / 8) >= 256) {
    im2col_rows_kernel<<<N * Ho, 256, row_smem, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)col, H, W, C, Ho, Wo, KH,
                                                          KW, stride, pad_h, pad_w, RP, Kp);
    return (int)cudaGetLastError();
  }
  const long total = (long)N * Ho * Wo * (Kp / 8);
  long grid = (total + 255) / 256;
  const long cap = (long)axh::sm_count() * 16;
  if (grid > cap) grid = cap;
  im2col_nhwc_kernel<<<(int)grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)col, N, H, W, C, Ho, Wo, KH, KW,
                                                    stride, pad_h, pad_w, RP, Kp);
  return (int)cudaGetLastError();
}
