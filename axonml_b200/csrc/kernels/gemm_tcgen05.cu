// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with
// the accumulator in TMEM -> tcgen05.ld epilogue (bias, activation, optional second output) ->
// TMA store.  One CTA per SM; the accumulator is double-buffered in TMEM so that the epilogue of
// tile i overlaps the main loop of tile i+1.
//
//   C[M,N] = act(A[M,K] * B[K,N] + bias[N])
//
// Operand layouts ("major" = which logical dimension is contiguous in memory):
//   A: K-major  = row-major [M,K]          MN-major = row-major [K,M]   (A given transposed)
//   B: K-major  = row-major [N,K] (Linear) MN-major = row-major [K,N]
// which covers forward (A K, B K), dgrad (A K, B MN) and wgrad (A MN, B MN) of a Linear layer
// without materialising a transpose.
//
// Replaces the reference's CPU FusedLinear (crates/axonml-fusion/src/linear.rs:138-164), the
// Linear forward (crates/axonml-nn/src/layers/linear.rs:104-140) and its cuBLAS sgemm island
// (crates/axonml-core/src/backends/cuda.rs:413-451).
#include "common.cuh"

namespace {

using namespace ax;

constexpr int BM = 128;
constexpr int BK = 64;       // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..5: epilogue
constexpr int kEpiWarps = 4;
constexpr int kStageBufBytes = 32 * 128;  // 32 rows x 64 bf16 staging tile for the TMA store
// Estimated cost of one CTA-pair tile (256 x 256, 256 x 128) in the units of the tile chooser.
constexpr double kPairCost256 = 1.87;
constexpr double kPairCost128 = 1.55;

struct GemmParams {
  int M, N, K;
  const void* bias;  // per output column
  int bias_kind;     // 0 none, 1 fp32, 2 bf16
  int act;           // ax::Act applied to C
  int has_aux;       // also store the pre-activation (A*B + bias) through map_aux
  int* status;
};

template <int BN>
struct Cfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
  static constexpr int kSmem =
      1024 /*alignment slack*/ + kStages * kStage + kEpiWarps * 2 * kStageBufBytes + 256;
};

template <int BN, int A_MN, int B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c,
                 const __grid_constant__ CUtensorMap map_aux, const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* epi_base = smem + C::kStages * C::kStage;
  uint64_t* bars = (uint64_t*)(epi_base + kEpiWarps * 2 * kStageBufBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + C::kStages;         // [kStages]
  uint64_t* tfull_bar = bars + 2 * C::kStages;     // [2]
  uint64_t* tempty_bar = bars + 2 * C::kStages + 2;  // [2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * C::kStages + 4);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], kEpiWarps);
    }
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_c);
  }
  if (warp == 1) {
    tmem_alloc<C::kTmemCols>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Tile order: groups of 8 M-blocks sweep all N-blocks, so that concurrently running CTAs
  // share A and B tiles through L2.
  auto tile_coords = [&](int t, int& mb, int& nb) {
    constexpr int G = 8;
    int per_group = G * num_n;
    int g = t / per_group;
    int first_m = g * G;
    int gsz = min(G, num_m - first_m);
    int r = t - g * per_group;
    mb = first_m + r % gsz;
    nb = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 100)) break;
          uint8_t* sa = stage_base + s * C::kStage;
          uint8_t* sb = sa + C::kStageA;
          mbar_expect_tx(&full_bar[s], C::kStage);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &map_a, &full_bar[s], m0 + j * 64, k0);
          } else {
            tma_load_2d(sa, &map_a, &full_bar[s], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &map_b, &full_bar[s], n0 + j * 64, k0);
          } else {
            tma_load_2d(sb, &map_b, &full_bar[s], k0, n0);
          }
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        if (*dead) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // One thread feeds the tensor core, so its instruction stream sits on the critical path:
      // the shared-memory descriptors of stage 0 are built once and every MMA only adds the
      // (16-byte-unit) offset of its stage and k step to them.
      constexpr uint32_t idesc = umma_idesc_f16(1, BM, BN, A_MN, B_MN);
      const uint32_t sa0 = smem_u32(stage_base);
      const uint64_t da0 = A_MN ? umma_desc_sw128(sa0, BK * 128, 1024) : umma_desc_sw128(sa0, 16, 1024);
      const uint64_t db0 = B_MN ? umma_desc_sw128(sa0 + C::kStageA, BK * 128, 1024)
                                : umma_desc_sw128(sa0 + C::kStageA, 16, 1024);
      constexpr uint32_t kStepA = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
      constexpr uint32_t kStepB = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, dead, p.status, 200)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, dead, p.status, 201)) break;
          tc_fence_after();
          const uint64_t soff = (uint64_t)((uint32_t)(s * C::kStage) >> 4);
          const uint64_t da = da0 + soff, db = db0 + soff;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            umma_f16_ss(d_tmem, da + (uint64_t)(k * kStepA), db + (uint64_t)(k * kStepB), idesc, accum);
            accum = 1;
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        umma_commit(&tfull_bar[acc]);  // accumulator complete
        if (*dead) break;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int ew = warp - 2;           // staging-buffer owner index
    uint8_t* stg = epi_base + ew * 2 * kStageBufBytes;
    int buf = 0;
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      int mb, nb;
      tile_coords(t, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      bool ok = mbar_wait(&tfull_bar[acc], acc_ph, dead, p.status, 300);
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
          // all of this warp's TMEM reads for the tile are done: hand the accumulator back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        }
        const int ncol0 = n0 + ch * 64;
        if (ncol0 >= p.N) continue;  // fully out-of-range chunk (warp-uniform)
        add_bias_chunk(r, p.bias, p.bias_kind, ncol0, p.N);
        const int passes = p.has_aux ? 2 : 1;
        for (int pass = 0; pass < passes; ++pass) {
          const bool is_aux = p.has_aux && pass == 0;
          if (!is_aux) apply_act_chunk(r, p.act);      // the aux output keeps the pre-activation values
          uint8_t* dst = stg + buf * kStageBufBytes;
          // the bulk store that last read this buffer must have finished reading it
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
          if (lane == 0) {
            tma_store_2d(is_aux ? &map_aux : &map_c, dst, ncol0, m0 + q * 32);
            tma_store_commit();
          }
          buf ^= 1;
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<C::kTmemCols>(tmem_base);
}

// ------------------------------------------------------------------ CTA-pair kernel
// Two CTAs of a cluster share one 256 x BN output tile (tcgen05 cta_group::2).  CTA r of the pair
// loads rows [128 r, 128 r + 128) of the A tile and columns [BN/2 r, BN/2 (r+1)) of the B tile with
// plain TMA loads of its own (no multicast), so a k step of 64 costs 16 KB + BN/2 x 128 B of
// shared-memory fill per SM for the same 128 x BN x 64 of math: two thirds of the one-CTA kernel's
// fill at BN = 256, which leaves room for six stages.  The even CTA issues every MMA (M = 256)
// and signals both CTAs' barriers through the commit; each CTA drains its own 128 accumulator
// rows.  Barriers: full[s] lives in the leader and counts the bytes of both CTAs' loads;
// empty[s] and tfull[a] exist in both CTAs; tempty[a] lives in the leader and collects the
// epilogue warps of both.
template <int BN>
struct PairCfg {
  static constexpr int kStageA = BM * BK * 2;          // this CTA's 128 rows of A
  static constexpr int kStageB = (BN / 2) * BK * 2;    // this CTA's half of the B tile
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 6 : 8;
  // The whole TMEM of both SMs: an allocation of part of it could land at different columns in
  // the two CTAs when another kernel holds TMEM on one of the SMs, and the MMA addresses both
  // accumulators by one column number.
  static constexpr int kTmemCols = 512;
  static constexpr int kSmem =
      1024 + kStages * kStage + kEpiWarps * 2 * kStageBufBytes + 256;
};

template <int BN, int A_MN, int B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_c,
                      const __grid_constant__ CUtensorMap map_aux, const GemmParams p) {
  using C = PairCfg<BN>;
  constexpr int HB = BN / 2;
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
  const uint32_t crank = cluster_ctarank();      // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  constexpr int PM = 2 * BM;
  const int num_m = (p.M + PM - 1) / PM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 2 * kEpiWarps);
    }
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_c);
  }
  if (warp == 1) {
    tmem_alloc_pair<C::kTmemCols>(tmem_slot);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();   // both CTAs' barriers are initialised before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int t, int& mb, int& nb) {
    constexpr int G = 4;
    int per_group = G * num_n;
    int g = t / per_group;
    int first_m = g * G;
    int gsz = min(G, num_m - first_m);
    int r = t - g * per_group;
    mb = first_m + r % gsz;
    nb = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int t = pair_id; t < num_tiles; t += num_pairs) {
        int mb, nb;
        tile_coords(t, mb, nb);
        const int m0 = mb * PM + (int)crank * BM, n0 = nb * BN + (int)crank * HB;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 110)) break;
          uint8_t* sa = stage_base + s * C::kStage;
          uint8_t* sb = sa + C::kStageA;
          if (crank == 0) mbar_expect_tx(&full_bar[s], 2 * C::kStage);
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[s]), 0);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d_pair(sa + j * (BK * 128), &map_a, fb, m0 + j * 64, k0);
          } else {
            tma_load_2d_pair(sa, &map_a, fb, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < HB / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), &map_b, fb, n0 + j * 64, k0);
          } else {
            tma_load_2d_pair(sb, &map_b, fb, k0, n0);
          }
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        if (*dead) break;
      }
      // Tail: every arrive the leader's commits still owe this CTA's empty barriers must land
      // before the CTA may leave.
      for (int i = 0; i < C::kStages && !*dead; ++i) {
        if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 111)) break;
        if (++s == C::kStages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && crank == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(1, PM, BN, A_MN, B_MN);
      const uint32_t sa0 = smem_u32(stage_base);
      const uint64_t da0 = A_MN ? umma_desc_sw128(sa0, BK * 128, 1024) : umma_desc_sw128(sa0, 16, 1024);
      const uint64_t db0 = B_MN ? umma_desc_sw128(sa0 + C::kStageA, BK * 128, 1024)
                                : umma_desc_sw128(sa0 + C::kStageA, 16, 1024);
      constexpr uint32_t kStepA = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
      constexpr uint32_t kStepB = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int t = pair_id; t < num_tiles; t += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, dead, p.status, 210)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, dead, p.status, 211)) break;
          tc_fence_after();
          const uint64_t soff = (uint64_t)((uint32_t)(s * C::kStage) >> 4);
          const uint64_t da = da0 + soff, db = db0 + soff;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            umma_f16_ss_pair(d_tmem, da + (uint64_t)(k * kStepA), db + (uint64_t)(k * kStepB), idesc, accum);
            accum = 1;
          }
          umma_commit_pair(&empty_bar[s]);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        umma_commit_pair(&tfull_bar[acc]);
        if (*dead) break;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps per CTA)
    const int q = warp & 3;
    const int ew = warp - 2;
    uint8_t* stg = epi_base + ew * 2 * kStageBufBytes;
    const uint32_t tempty_leader0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    int buf = 0;
    int it = 0;
    for (int t = pair_id; t < num_tiles; t += num_pairs, ++it) {
      int mb, nb;
      tile_coords(t, mb, nb);
      const int m0 = mb * PM + (int)crank * BM, n0 = nb * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      bool ok = mbar_wait(&tfull_bar[acc], acc_ph, dead, p.status, 310);
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
          if (lane == 0) mbar_arrive_cluster(tempty_leader0 + acc * 8);
        }
        const int ncol0 = n0 + ch * 64;
        if (ncol0 >= p.N) continue;
        if (m0 + q * 32 >= p.M) continue;   // rows past the matrix (warp-uniform)
        add_bias_chunk(r, p.bias, p.bias_kind, ncol0, p.N);
        const int passes = p.has_aux ? 2 : 1;
        for (int pass = 0; pass < passes; ++pass) {
          const bool is_aux = p.has_aux && pass == 0;
          if (!is_aux) apply_act_chunk(r, p.act);
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
          if (lane == 0) {
            tma_store_2d(is_aux ? &map_aux : &map_c, dst, ncol0, m0 + q * 32);
            tma_store_commit();
          }
          buf ^= 1;
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // Neither CTA may leave (or free TMEM) while the other can still read its shared memory, write
  // its accumulator or signal its barriers.
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair<C::kTmemCols>(tmem_base);
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* ptr;
  uint64_t d0, d1, ld;
  uint32_t b0, b1;
};

int make_map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {ld_elems * 2};
  uint32_t box[2] = {box_inner, box_outer};
  return axh::encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BN, int A_MN, int B_MN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
           const CUtensorMap& maux, const GemmParams& p, int max_ctas, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = num_tiles < max_ctas ? num_tiles : max_ctas;
  if (grid < 1) grid = 1;
  kern<<<grid, kThreads, C::kSmem, stream>>>(ma, mb, mc, maux, p);
  return (int)cudaGetLastError();
}

template <int BN>
int dispatch_major(int a_mn, int b_mn, const CUtensorMap& ma, const CUtensorMap& mb,
                   const CUtensorMap& mc, const CUtensorMap& maux, const GemmParams& p,
                   int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch<BN, 0, 0>(ma, mb, mc, maux, p, max_ctas, stream);
  if (!a_mn && b_mn) return launch<BN, 0, 1>(ma, mb, mc, maux, p, max_ctas, stream);
  if (a_mn && !b_mn) return launch<BN, 1, 0>(ma, mb, mc, maux, p, max_ctas, stream);
  return launch<BN, 1, 1>(ma, mb, mc, maux, p, max_ctas, stream);
}

// ---- CTA-pair launch: a cluster of two CTAs per tile, as many pairs as the device can hold at once.
template <int BN, int A_MN, int B_MN>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                const CUtensorMap& maux, const GemmParams& p, int max_ctas, cudaStream_t stream) {
  using C = PairCfg<BN>;
  auto kern = gemm_bf16_pair_kernel<BN, A_MN, B_MN>;
  static int max_pairs[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs[dev] == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) return (int)e;
    cfg.gridDim = dim3(2 * axh::sm_count(), 1, 1);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, (const void*)kern, &cfg);
    if (e != cudaSuccess) return (int)e;
    if (n < 1) return -3;
    max_pairs[dev] = n;
  }
  if (p.M == 0) return max_pairs[dev];   // capacity query, nothing launched
  const int num_tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
  int pairs = max_pairs[dev];
  if (max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (num_tiles < pairs) pairs = num_tiles;
  if (pairs < 1) pairs = 1;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  return (int)cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, maux, p);
}

template <int BN>
int dispatch_major_pair(int a_mn, int b_mn, const CUtensorMap& ma, const CUtensorMap& mb,
                        const CUtensorMap& mc, const CUtensorMap& maux, const GemmParams& p,
                        int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_pair<BN, 0, 0>(ma, mb, mc, maux, p, max_ctas, stream);
  if (!a_mn && b_mn) return launch_pair<BN, 0, 1>(ma, mb, mc, maux, p, max_ctas, stream);
  if (a_mn && !b_mn) return launch_pair<BN, 1, 0>(ma, mb, mc, maux, p, max_ctas, stream);
  return launch_pair<BN, 1, 1>(ma, mb, mc, maux, p, max_ctas, stream);
}

int g_pair_mode = -1;   // -1 choose per shape, 0 one CTA per tile always, 1 CTA pairs whenever legal

// CTA pairs the current device runs at once (clusters of two need both SMs in one GPC, so this can
// be below half the SM count).  Negative: the query failed.
int pair_capacity() {
  static int cap[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cap[dev] == 0) {
    CUtensorMap dummy = {};
    GemmParams q = {};
    int n = launch_pair<256, 0, 0>(dummy, dummy, dummy, dummy, q, 0, nullptr);
    cap[dev] = n > 0 ? n : -1;
  }
  return cap[dev];
}

}  // namespace

// Tile-shape policy of ax_gemm_bf16: -1 (default) chooses per shape, 0 forces one CTA per tile,
// 1 forces CTA pairs wherever the shape allows them.  For benchmarks and tests.
AX_API void ax_gemm_set_pair_mode(int mode) { g_pair_mode = mode; }
AX_API int ax_gemm_pair_capacity() { return pair_capacity(); }

// C[M,N] (bf16, row stride ldc) = act(A*B + bias).  `a_mn` / `b_mn` select the operand layout
// (see the file header); lda / ldb are the row strides, in elements, of the matrices as stored.
// `aux` (may be null) receives the pre-activation.  `bn_hint` forces the N tile (0 = choose).
// `max_ctas` limits the persistent grid (0 = one per SM), so that a concurrent kernel on another
// stream keeps some SMs.  Returns a cudaError_t value, or -1 for an unsupported argument.
AX_API int ax_gemm_bf16(const void* A, const void* B, void* Cout, void* aux, const void* bias,
                        int bias_kind, int act, int M, int N, int K, int lda, int ldb, int ldc,
                        int a_mn, int b_mn, int bn_hint, int max_ctas, int* status,
                        cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % 8)) return -1;
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)Cout | (uintptr_t)aux) & 15) return -1;
  int sms = axh::sm_count();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;

  // Tile choice: the lowest estimated time, waves x per-tile cost.  Costs are in units of half a
  // 128 x 256 one-CTA tile and come from timings of the four kernels on full waves.
  int BN = bn_hint;
  bool pair = false;
  const int pair_cap = (g_pair_mode != 0 && M > BM && N >= 128) ? pair_capacity() : 0;
  const bool pair_legal = pair_cap > 0;
  if (BN != 64 && BN != 128 && BN != 256) {
    if (N <= 64) {
      BN = 64;
    } else {
      auto waves = [&](int bm, int bn, int ctas) {
        long tiles = (long)((M + bm - 1) / bm) * ((N + bn - 1) / bn);
        return (double)((tiles + ctas - 1) / ctas);
      };
      const int pairs = max_ctas / 2 < pair_cap ? (max_ctas / 2 > 0 ? max_ctas / 2 : 1) : pair_cap;
      double best = 1e30;
      auto consider = [&](double cost, int bn, bool pr) {
        if (cost < best) { best = cost; BN = bn; pair = pr; }
      };
      if (g_pair_mode != 1 || !pair_legal) {
        if (N > 128) consider(waves(BM, 256, max_ctas) * 2.0, 256, false);
        consider(waves(BM, 128, max_ctas) * 1.45, 128, false);
      }
      if (g_pair_mode != 0 && pair_legal) {
        if (N > 128) consider(waves(2 * BM, 256, pairs) * kPairCost256, 256, true);
        consider(waves(2 * BM, 128, pairs) * kPairCost128, 128, true);
      }
    }
  } else {
    pair = pair_legal && BN >= 128 && g_pair_mode == 1;
  }

  CUtensorMap ma, mb, mc, maux;
  int rc;
  if (a_mn)
    rc = make_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK);
  else
    rc = make_map_2d(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return 1000 + rc;
  if (b_mn)
    rc = make_map_2d(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
  else
    rc = make_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, (uint32_t)(pair ? BN / 2 : BN));
  if (rc) return 2000 + rc;
  rc = make_map_2d(&mc, Cout, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 32);
  if (rc) return 3000 + rc;
  if (aux) {
    rc = make_map_2d(&maux, aux, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 32);
    if (rc) return 4000 + rc;
  } else {
    maux = mc;
  }

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.bias = bias;
  p.bias_kind = bias ? bias_kind : 0;
  p.act = act;
  p.has_aux = aux ? 1 : 0;
  p.status = status;
  if (pair) {
    if (BN == 256) return dispatch_major_pair<256>(a_mn, b_mn, ma, mb, mc, maux, p, max_ctas, stream);
    return dispatch_major_pair<128>(a_mn, b_mn, ma, mb, mc, maux, p, max_ctas, stream);
  }
  switch (BN) {
    case 256: return dispatch_major<256>(a_mn, b_mn, ma, mb, mc, maux, p, max_ctas, stream);
    case 128: return dispatch_major<128>(a_mn, b_mn, ma, mb, mc, maux, p, max_ctas, stream);
    default: return dispatch_major<64>(a_mn, b_mn, ma, mb, mc, maux, p, max_ctas, stream);
  }
}
