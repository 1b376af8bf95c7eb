// Tensor-parallel GEMMs fused with their collective, one launch each, over NVLink peer memory:
//
//  MODE_AG  all-gather -> GEMM (column-parallel Linear with sequence-parallel input):
//           C[W*Tl, N] = act(concat_r(X_r)[W*Tl, K] * B[N, K]^T + bias).
//           A few "pusher" CTAs copy this rank's shard X_rank, 128 rows at a time, into slot `rank`
//           of every peer's gathered buffer (bulk loads into shared memory, bulk stores to the
//           peers' memory) and raise a per-chunk flag in the peer's memory.  The GEMM CTAs start on the local shard at once and take the other
//           shards in ring order; the TMA producer of a tile waits for the flag of the chunk it
//           is about to read, so the transfer overlaps the math chunk by chunk.  TMA reads only
//           this GPU's own memory.
//
//  MODE_RS  GEMM -> reduce-scatter (row-parallel Linear with sequence-parallel output):
//           out[Tl, N] = act(sum_r (X_r[W*Tl, Kl] * B_r[N, Kl]^T)[rows of this rank] + bias).
//           Every rank computes its partial product tile by tile, the destination shard after
//           its own first and its own shard last, and the epilogue sends each finished tile
//           (bf16, TMEM -> shared memory -> tensor bulk store) into the destination rank's staging
//           slot for this source, then raises a per-tile flag there.  The tiles of the rank's own
//           rows come last: their epilogue waits for the peers' flags, adds the W-1 staged copies
//           to the fp32 accumulator and writes the result.  Deterministic (no floating-point atomics).
//
// Flags hold the call's epoch and only grow; a rank tells its peers "call e consumed" at the end
// of the kernel, and the next call waits for that before it overwrites peer memory.  Every wait
// is bounded and reports through the status word.
//
// Replaces crates/axonml-distributed/src/fsdp.rs:463-483 (ColumnParallelLinear: all_gather then
// matmul) and fsdp.rs:550-591 (RowParallelLinear: matmul then all_reduce) of the reference, which
// run on a CPU mock backend.
#include "comm.cuh"

namespace {
using namespace ax;
using namespace axc;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;      // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..5: epilogue
constexpr int kEpiWarps = 4;
constexpr int kStageBufBytes = 32 * 128;
constexpr int kSigDone = 0;        // [kMaxRanks] "rank p consumed call e"
constexpr int kSigCounter = 8;     // local: CTAs of this rank that finished the call
constexpr int kSigFlags = 16;      // [world][max_tiles][4] chunk / tile flags (RS: one per epilogue warp)
constexpr int kFlagsPerTile = 4;

enum { MODE_AG = 0, MODE_RS = 1 };

struct CommParams {
  int M, N, K;           // the GEMM as computed on this rank (M = world * Tl)
  int Tl;                // rows per shard
  int rank, world;
  uint32_t epoch;
  uint32_t* sig[kMaxRanks];
  uint8_t* sym[kMaxRanks];   // AG: gathered X [world][Tl][K]; RS: staging [world][Tl][N]  (bf16)
  uint8_t* sym_mc;           // multicast mapping of `sym`, or null
  const uint8_t* x_local;    // AG: this rank's shard [Tl][K]
  uint8_t* out;              // RS: result [Tl][N] bf16
  const void* bias;
  int bias_kind;             // 0 none, 1 fp32, 2 bf16
  int act;
  int pushers;               // AG: CTAs that only copy
  int max_tiles;             // flags per source rank
  int* status;
  unsigned long long* trace; // optional timeline [grid][kTraceSlots] of globaltimer stamps, or null
};

// Timeline slots per CTA: 0 kernel start, 1 start-of-call wait done, then four per tile
// (accumulator ready, peers' flags seen, epilogue done, MMA issued), 62 epilogue loop done, 63 end.
constexpr int kTraceSlots = 64;
__device__ __forceinline__ void trace_at(const CommParams& p, int slot) {
  if (p.trace != nullptr && slot < kTraceSlots) p.trace[(long)blockIdx.x * kTraceSlots + slot] = globaltimer_ns();
}

template <int BN>
struct Cfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmem = 1024 + kStages * kStage + kEpiWarps * 2 * kStageBufBytes + 256;
};

__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// Tile t of this CTA's schedule -> (shard, m block inside the shard, n block).
struct TileMap {
  int mbs, num_n, rank, world, first;   // first: offset of the first shard relative to `rank`
  __device__ __forceinline__ void coords(int t, int& ring_pos, int& shard, int& mb, int& nb) const {
    const int per_shard = mbs * num_n;
    ring_pos = t / per_shard;
    const int r = t - ring_pos * per_shard;
    mb = r / num_n;
    nb = r - mb * num_n;
    shard = (rank + first + ring_pos) % world;
  }
};

// This rank's shard -> slot `rank` of every peer's gathered buffer, one 128-row chunk at a time.
// One thread runs the whole copy as an asynchronous pipeline: bulk loads bring 16 KB pieces of the
// local rows into shared memory, bulk stores send each piece to every peer (per-thread stores to a
// peer are limited by the few outstanding writes an SM tracks; the bulk engine is not).  When the
// stores of a chunk have completed, the chunk's flag is raised in every peer's memory.
constexpr int kPushPiece = 16384;
constexpr int kPushStages = 12;      // 192 KB of shared memory
constexpr int kPushAhead = 4;        // loads in flight; the other stages hold pieces being sent

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)),
               "r"(bytes)
               : "memory");
}

// NVSwitch variant for more than two ranks: one multimem store delivers 16 bytes to every rank, so
// the shard leaves this GPU once instead of W-1 times.  Thread 0 keeps the bulk loads running, all
// threads forward from shared memory.
__device__ void push_shard_multimem(const CommParams& p, int pusher, int npushers, uint8_t* buf, uint64_t* full,
                                    volatile int* dead) {
  const int chunks = p.Tl / BM;
  const long row_bytes = (long)p.K * 2;
  const long chunk_bytes = (long)BM * row_bytes;
  const int pieces = (int)(chunk_bytes / kPushPiece);
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_ok = 1;
    *dead = 0;
    for (int i = 0; i < kPushStages; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank)
    if (!wait_ge<true>(p.sig[p.rank] + kSigDone + threadIdx.x, p.epoch - 1, p.status, 802)) s_ok = 0;
  __syncthreads();
  if (!s_ok) return;
  int my_chunks = 0;
  for (int c = pusher; c < chunks; c += npushers) ++my_chunks;
  const long total = (long)my_chunks * pieces;
  auto piece_src = [&](long i) {
    const int c = pusher + (int)(i / pieces) * npushers;
    return p.x_local + (long)c * chunk_bytes + (i % pieces) * (long)kPushPiece;
  };
  if (threadIdx.x == 0) {
    for (long i = 0; i < kPushStages - 1 && i < total; ++i) {
      mbar_expect_tx(&full[i % kPushStages], kPushPiece);
      bulk_load_1d(buf + (i % kPushStages) * kPushPiece, piece_src(i), kPushPiece, &full[i % kPushStages]);
    }
  }
  for (long i = 0; i < total; ++i) {
    const int st = (int)(i % kPushStages);
    if (threadIdx.x == 0) {
      const long nx = i + kPushStages - 1;      // its stage was drained before the last barrier
      if (nx < total) {
        mbar_expect_tx(&full[nx % kPushStages], kPushPiece);
        bulk_load_1d(buf + (nx % kPushStages) * kPushPiece, piece_src(nx), kPushPiece, &full[nx % kPushStages]);
      }
    }
    const bool ok = mbar_wait(&full[st], (uint32_t)((i / kPushStages) & 1), dead, p.status, 803);
    if (!__syncthreads_and(ok)) return;
    const int c = pusher + (int)(i / pieces) * npushers;
    const long dst_off = ((long)p.rank * p.Tl + (long)c * BM) * row_bytes + (i % pieces) * (long)kPushPiece;
    const uint32_t sbase = smem_u32(buf + st * kPushPiece);
#pragma unroll 4
    for (int j = threadIdx.x; j < kPushPiece / 16; j += kThreads) {
      uint4 v;
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(sbase + j * 16));
      multimem_st_b32x4(p.sym_mc + dst_off + (long)j * 16, v);
    }
    const bool chunk_done = (i % pieces) == pieces - 1;
    if (chunk_done) __threadfence_system();
    __syncthreads();
    if (chunk_done && (int)threadIdx.x < p.world && (int)threadIdx.x != p.rank)
      st_release_sys(p.sig[threadIdx.x] + kSigFlags + (p.rank * p.max_tiles + c) * kFlagsPerTile, p.epoch);
  }
}

__device__ void push_shard(const CommParams& p, int pusher, int npushers, uint8_t* smem) {
  const int chunks = p.Tl / BM;
  const long row_bytes = (long)p.K * 2;
  const long chunk_bytes = (long)BM * row_bytes;            // a multiple of 16 KB (K % 64 == 0)
  const int pieces = (int)(chunk_bytes / kPushPiece);
  uint8_t* buf = smem;                                                       // [stages][piece]
  uint64_t* full = (uint64_t*)(smem + kPushStages * kPushPiece);             // [stages]
  volatile int* dead = (volatile int*)(full + kPushStages);
  if (p.sym_mc != nullptr && p.world > 2) {
    push_shard_multimem(p, pusher, npushers, buf, full, dead);
    return;
  }
  if (threadIdx.x != 0) return;
  *dead = 0;
  for (int i = 0; i < kPushStages; ++i) mbar_init(&full[i], 1);
  mbar_fence_init();
  // the peers must have finished reading what the previous call put there
  for (int q = 0; q < p.world; ++q)
    if (q != p.rank && !wait_ge<true>(p.sig[p.rank] + kSigDone + q, p.epoch - 1, p.status, 800)) return;
  int my_chunks = 0;
  for (int c = pusher; c < chunks; c += npushers) ++my_chunks;
  const long total = (long)my_chunks * pieces;               // pieces this CTA forwards, in order
  auto piece_src = [&](long i) {
    const int c = pusher + (int)(i / pieces) * npushers;
    return p.x_local + (long)c * chunk_bytes + (i % pieces) * (long)kPushPiece;
  };
  for (long i = 0; i < kPushAhead && i < total; ++i) {
    mbar_expect_tx(&full[i % kPushStages], kPushPiece);
    bulk_load_1d(buf + (i % kPushStages) * kPushPiece, piece_src(i), kPushPiece, &full[i % kPushStages]);
  }
  for (long i = 0; i < total; ++i) {
    const int st = (int)(i % kPushStages);
    if (!mbar_wait(&full[st], (uint32_t)((i / kPushStages) & 1), dead, p.status, 801)) break;
    const int c = pusher + (int)(i / pieces) * npushers;
    const long dst_off = ((long)p.rank * p.Tl + (long)c * BM) * row_bytes + (i % pieces) * (long)kPushPiece;
    for (int q = 1; q < p.world; ++q)
      bulk_store_1d(p.sym[(p.rank + q) % p.world] + dst_off, buf + st * kPushPiece, kPushPiece);
    tma_store_commit();
    // the stage that piece i + kPushAhead will use was last read by the stores of piece
    // i + kPushAhead - kPushStages: allow the more recent groups to stay in flight
    tma_store_wait_read<kPushStages - kPushAhead>();
    const long nx = i + kPushAhead;
    if (nx < total) {
      mbar_expect_tx(&full[nx % kPushStages], kPushPiece);
      bulk_load_1d(buf + (nx % kPushStages) * kPushPiece, piece_src(nx), kPushPiece, &full[nx % kPushStages]);
    }
    if ((i % pieces) == pieces - 1) {
      tma_store_wait<0>();                 // the chunk has landed on every peer
      fence_proxy_async_global();
      __threadfence_system();
      for (int q = 0; q < p.world; ++q)
        if (q != p.rank) st_release_sys(p.sig[q] + kSigFlags + (p.rank * p.max_tiles + c) * kFlagsPerTile, p.epoch);
    }
  }
  tma_store_wait<0>();
}

// Last CTA of the launch tells every peer that this rank has consumed the call.
__device__ __forceinline__ void finish_call(const CommParams& p) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* counter = p.sig[p.rank] + kSigCounter;
    const uint32_t old = atomicAdd(counter, 1u);
    if (old + 1 == p.epoch * gridDim.x) {
      for (int q = 0; q < p.world; ++q)
        if (q != p.rank) st_release_sys(p.sig[q] + kSigDone + p.rank, p.epoch);
    }
  }
}

// RS staging buffer of a rank: [source rank][128-row block][64-column chunk][epilogue warp] pieces
// of 4 KB, each the shared-memory image (128-byte swizzle) of a 32 x 64 bf16 sub-tile.
__device__ __forceinline__ long stage_off(const CommParams& p, const TileMap& tm, int src, int mb, int chunk, int ew) {
  const int nchunks = (p.N + 63) >> 6;
  return ((((long)src * tm.mbs + mb) * nchunks + chunk) * kEpiWarps + ew) * (long)kStageBufBytes;
}

struct DstMaps { CUtensorMap m[kMaxRanks]; };     // RS: every rank's staging buffer as [world*Tl, N]

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_local,
                 const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                 const __grid_constant__ DstMaps dst_maps, const CommParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  if (MODE == MODE_AG && (int)blockIdx.x < p.pushers) {
    push_shard(p, blockIdx.x, p.pushers, smem);
    finish_call(p);
    return;
  }
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
  const int first_cta = MODE == MODE_AG ? p.pushers : 0;
  const int cta = blockIdx.x - first_cta;
  const int ncta = gridDim.x - first_cta;

  TileMap tm;
  tm.mbs = p.Tl / BM;
  tm.num_n = (p.N + BN - 1) / BN;
  tm.rank = p.rank;
  tm.world = p.world;
  tm.first = MODE == MODE_AG ? 0 : 1;          // AG: own shard first; RS: own shard last
  const int num_tiles = p.world * tm.mbs * tm.num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  uint32_t* my_flags = p.sig[p.rank] + kSigFlags;

  if (threadIdx.x == 0) {
    trace_at(p, 0);
    *dead = 0;
    for (int i = 0; i < C::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], kEpiWarps); }
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
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
      for (int t = cta; t < num_tiles; t += ncta) {
        int ring_pos, shard, mb, nb;
        tm.coords(t, ring_pos, shard, mb, nb);
        const CUtensorMap* ma = &map_a;
        int m0 = shard * p.Tl + mb * BM;
        if (MODE == MODE_AG) {
          if (shard == p.rank) {
            ma = &map_a_local;
            m0 = mb * BM;
          } else {
            // the chunk must have arrived; then order the peer's writes before the TMA reads
            if (!wait_ge<true>(my_flags + (shard * p.max_tiles + mb) * kFlagsPerTile, p.epoch, p.status, 810)) { *dead = 1; break; }
            fence_proxy_async_global();
          }
        }
        const int n0 = nb * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 811)) break;
          uint8_t* sa = stage_base + s * C::kStage;
          mbar_expect_tx(&full_bar[s], C::kStage);
          tma_load_2d(sa, ma, &full_bar[s], kb * BK, m0);
          tma_load_2d(sa + C::kStageA, &map_b, &full_bar[s], kb * BK, n0);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
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
      for (int t = cta; t < num_tiles; t += ncta, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, dead, p.status, 820)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, dead, p.status, 821)) break;
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
        trace_at(p, 2 + 4 * it + 3);
        if (*dead) break;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;
    const int ew = warp - 2;
    uint8_t* stg = epi_base + ew * 2 * kStageBufBytes;
    int buf = 0, it = 0;
    bool ok = true;
    // lane 0: remote tiles [pend_first, pend_first + pend_n * ncta) of ring phase `pend_shard` whose
    // flags are still owed.  A completion wait on stores to a peer costs a round trip under load,
    // so flags go out once per ring phase (the owner needs them only for its own rows, which it
    // computes last), one tile into the next phase so that the wait overlaps that tile's work.
    int pend_first = 0, pend_n = 0, pend_shard = -1;
    auto release_flags = [&](int first, int n) {
      fence_proxy_async_global();
      __threadfence_system();
      for (int i = 0; i < n; ++i) {
        int rp, sh, mb2, nb2;
        tm.coords(first + i * ncta, rp, sh, mb2, nb2);
        st_release_sys(p.sig[sh] + kSigFlags + ((p.rank * p.max_tiles + mb2 * tm.num_n + nb2) * kFlagsPerTile + ew), p.epoch);
      }
    };
    if (MODE == MODE_RS) {
      // peers must have consumed the previous call before their staging slots are overwritten
      // (every warp checks for itself: no barrier that a timed-out warp could leave hanging)
      bool w_ok = true;
      if (lane < p.world && lane != p.rank) w_ok = wait_ge<true>(p.sig[p.rank] + kSigDone + lane, p.epoch - 1, p.status, 830);
      ok = __all_sync(0xffffffffu, w_ok);
      if (!ok) *dead = 1;      // the producer and MMA warps stop at their next wait
    }
    if (ew == 0 && lane == 0) trace_at(p, 1);
    for (int t = cta; t < num_tiles && ok; t += ncta, ++it) {
      int ring_pos, shard, mb, nb;
      tm.coords(t, ring_pos, shard, mb, nb);
      const int m0 = shard * p.Tl + mb * BM, n0 = nb * BN;
      const int acc = it & 1;
      ok = mbar_wait(&tfull_bar[acc], (it >> 1) & 1, dead, p.status, 831);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (ew == 0 && lane == 0) trace_at(p, 2 + 4 * it);
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
        const int ncol0 = n0 + ch * 64;
        if (ncol0 >= p.N) continue;
        if (MODE == MODE_AG) {
          add_bias_chunk(r, p.bias, p.bias_kind, ncol0, p.N);
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
          if (lane == 0) {
            tma_store_2d(&map_c, dst, ncol0, m0 + q * 32);
            tma_store_commit();
          }
          buf ^= 1;
        } else if (shard != p.rank) {
          // partial tile -> staging slot `rank` on the rank that owns these rows: the warp's
          // 32 x 64 sub-tile is staged in shared memory and sent as one contiguous 4 KB bulk
          // store (the staging buffer is tile-ordered; row-strided 128-byte writes over NVLink
          // ran at a third of the rate)
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
            bulk_store_1d(p.sym[shard] + stage_off(p, tm, p.rank, mb, ncol0 >> 6, ew), dst, kStageBufBytes);
            tma_store_commit();
          }
          buf ^= 1;
        } else {
          // a tile of this rank's own rows (scheduled last): add the peers' staged partial tiles
          // to the fp32 accumulator and write the finished output; nothing is staged locally
          if (ch == 0) {
            // the flag still owed for the last remote tile must go out first: the peers' own-row
            // tiles wait for it exactly as this one waits for theirs
            if (lane == 0 && pend_n > 0) {
              tma_store_wait<0>();
              release_flags(pend_first, pend_n);
              pend_n = 0;
            }
            __syncwarp();
            bool w_ok = true;       // lane l: the same quarter of this tile as sent by rank l
            if (lane < p.world && lane != p.rank)
              w_ok = wait_ge<true>(my_flags + ((lane * p.max_tiles + mb * tm.num_n + nb) * kFlagsPerTile + ew), p.epoch,
                                   p.status, 840);
            ok = __all_sync(0xffffffffu, w_ok);
            if (ew == 0 && lane == 0) trace_at(p, 2 + 4 * it + 1);
          }
          if (ok) {
            // two peers' pieces per round: sixteen 16-byte loads in flight per lane, so the W-1
            // dependent round trips to memory become (W-1)/2
            for (int j = 1; j < p.world; j += 2) {
              const int s0 = (p.rank + j) % p.world;
              const bool two = j + 1 < p.world;
              const int s1 = two ? (p.rank + j + 1) % p.world : s0;
              // the staged piece keeps the shared-memory image: row `lane`, 16-byte chunks swizzled
              const uint8_t* sp0 = p.sym[p.rank] + stage_off(p, tm, s0, mb, ncol0 >> 6, ew) + lane * 128;
              const uint8_t* sp1 = p.sym[p.rank] + stage_off(p, tm, s1, mb, ncol0 >> 6, ew) + lane * 128;
              uint4 u[8], v[8];
#pragma unroll
              for (int c = 0; c < 8; ++c) u[c] = ld_peer_v4(sp0 + ((c ^ (lane & 7)) << 4));
              if (two) {
#pragma unroll
                for (int c = 0; c < 8; ++c) v[c] = ld_peer_v4(sp1 + ((c ^ (lane & 7)) << 4));
              } else {
#pragma unroll
                for (int c = 0; c < 8; ++c) v[c] = make_uint4(0u, 0u, 0u, 0u);
              }
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const float2 x0 = unpack_bf16x2(u[c].x), x1 = unpack_bf16x2(u[c].y), x2 = unpack_bf16x2(u[c].z),
                             x3 = unpack_bf16x2(u[c].w);
                const float2 y0 = unpack_bf16x2(v[c].x), y1 = unpack_bf16x2(v[c].y), y2 = unpack_bf16x2(v[c].z),
                             y3 = unpack_bf16x2(v[c].w);
                r[c * 8 + 0] = __float_as_uint(__uint_as_float(r[c * 8 + 0]) + (x0.x + y0.x));
                r[c * 8 + 1] = __float_as_uint(__uint_as_float(r[c * 8 + 1]) + (x0.y + y0.y));
                r[c * 8 + 2] = __float_as_uint(__uint_as_float(r[c * 8 + 2]) + (x1.x + y1.x));
                r[c * 8 + 3] = __float_as_uint(__uint_as_float(r[c * 8 + 3]) + (x1.y + y1.y));
                r[c * 8 + 4] = __float_as_uint(__uint_as_float(r[c * 8 + 4]) + (x2.x + y2.x));
                r[c * 8 + 5] = __float_as_uint(__uint_as_float(r[c * 8 + 5]) + (x2.y + y2.y));
                r[c * 8 + 6] = __float_as_uint(__uint_as_float(r[c * 8 + 6]) + (x3.x + y3.x));
                r[c * 8 + 7] = __float_as_uint(__uint_as_float(r[c * 8 + 7]) + (x3.y + y3.y));
              }
            }
            add_bias_chunk(r, p.bias, p.bias_kind, ncol0, p.N);
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
            if (lane == 0) {
              tma_store_2d(&map_c, dst, ncol0, mb * BM + q * 32);
              tma_store_commit();
            }
            buf ^= 1;
          }
        }
      }
      if (ew == 0 && lane == 0) trace_at(p, 2 + 4 * it + 2);
      if (MODE == MODE_RS && shard != p.rank) {
        if (lane == 0) {
          if (pend_n > 0 && pend_shard != shard) {
            tma_store_wait<BN / 64>();          // all but this tile's groups: the last phase has landed
            release_flags(pend_first, pend_n);
            pend_n = 0;
          }
          if (pend_n == 0) { pend_first = t; pend_shard = shard; }
          ++pend_n;
        }
        __syncwarp();
      }
    }
    if (MODE == MODE_RS && lane == 0 && pend_n > 0) {
      tma_store_wait<0>();
      release_flags(pend_first, pend_n);
    }
    __syncwarp();
    if (ew == 0 && lane == 0) trace_at(p, 62);
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<C::kTmemCols>(tmem_base);
  if (threadIdx.x == 0) trace_at(p, 63);
  finish_call(p);
}

int make_map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {ld_elems * 2};
  uint32_t box[2] = {box_inner, box_outer};
  return axh::encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BN, int MODE>
int launch(const CUtensorMap& ma, const CUtensorMap& mal, const CUtensorMap& mb, const CUtensorMap& mc,
           const DstMaps& dm, const CommParams& p, int grid, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_comm_kernel<BN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, kThreads, C::kSmem, stream>>>(ma, mal, mb, mc, dm, p);
  return (int)cudaGetLastError();
}

}  // namespace

// Number of 32-bit slots a communicator's signal array needs for `max_tiles` flags per rank.
AX_API int ax_gemm_comm_signal_slots(int max_tiles) { return kSigFlags + kMaxRanks * max_tiles * kFlagsPerTile; }

// mode 0: C[world*Tl, N] = act(allgather(x_local)[world*Tl, K] * B[N, K]^T + bias); `sym` = gathered buffers,
//         `out` = C (row stride N).
// mode 1: out[Tl, N] = act(reduce_scatter(x[world*Tl, K] * B[N, K]^T) + bias); `sym` = staging buffers,
//         `x_local` = x.
// `grid` must be the same for every call on one communicator (the end-of-call counter relies on it)
// and must not exceed the SM count.  Requires Tl % 128 == 0, K % 64 == 0, N % 64 == 0.
// Diagnostic timeline: the launches that follow write globaltimer stamps of their phases into
// `buf` ([grid][64] 64-bit slots, zero-filled by the caller); null turns it off again.
static unsigned long long* g_trace_buf = nullptr;
AX_API void ax_gemm_comm_set_trace(void* buf) { g_trace_buf = (unsigned long long*)buf; }

AX_API int ax_gemm_comm(int mode, const void* x_local, const void* B, void* out, void* const* sym, void* sym_mc,
                        void* const* sig, const void* bias, int bias_kind, int act, int Tl, int N, int K,
                        int rank, int world, unsigned epoch, int max_tiles, int pushers, int grid, int* status,
                        cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || Tl <= 0 || Tl % BM || K % BK || N % 64 || grid > axh::sm_count()) return -1;
  const int BN = (N % 256 == 0) ? 256 : 128;
  if (N % BN) return -1;
  const int tiles_per_shard = (Tl / BM) * (mode == MODE_AG ? 1 : N / BN);
  if (tiles_per_shard > max_tiles) return -2;
  if (mode == MODE_AG && (pushers < 1 || pushers >= grid)) return -1;
  CommParams p;
  p.M = world * Tl; p.N = N; p.K = K; p.Tl = Tl; p.rank = rank; p.world = world; p.epoch = epoch;
  for (int i = 0; i < kMaxRanks; ++i) {
    p.sig[i] = i < world ? (uint32_t*)sig[i] : nullptr;
    p.sym[i] = i < world ? (uint8_t*)sym[i] : nullptr;
  }
  p.sym_mc = (uint8_t*)sym_mc;
  p.x_local = (const uint8_t*)x_local;
  p.out = (uint8_t*)out;
  p.bias = bias; p.bias_kind = bias ? bias_kind : 0; p.act = act;
  p.pushers = mode == MODE_AG ? pushers : 0;
  p.max_tiles = max_tiles;
  p.status = status;
  p.trace = g_trace_buf;
  CUtensorMap ma, mal, mb, mc;
  int rc;
  if (mode == MODE_AG) {
    rc = make_map_2d(&ma, sym[rank], (uint64_t)K, (uint64_t)world * Tl, (uint64_t)K, BK, BM);
    if (rc) return 1000 + rc;
    rc = make_map_2d(&mal, x_local, (uint64_t)K, (uint64_t)Tl, (uint64_t)K, BK, BM);
    if (rc) return 1100 + rc;
    rc = make_map_2d(&mc, out, (uint64_t)N, (uint64_t)world * Tl, (uint64_t)N, 64, 32);
    if (rc) return 3000 + rc;
  } else {
    rc = make_map_2d(&ma, x_local, (uint64_t)K, (uint64_t)world * Tl, (uint64_t)K, BK, BM);
    if (rc) return 1000 + rc;
    mal = ma;
    rc = make_map_2d(&mc, out, (uint64_t)N, (uint64_t)Tl, (uint64_t)N, 64, 32);
    if (rc) return 3000 + rc;
  }
  DstMaps dm;
  for (int i = 0; i < kMaxRanks; ++i) dm.m[i] = ma;
  if (mode == MODE_RS) {
    for (int i = 0; i < world; ++i) {
      rc = make_map_2d(&dm.m[i], sym[i], (uint64_t)N, (uint64_t)world * Tl, (uint64_t)N, 64, 32);
      if (rc) return 4000 + rc;
    }
  }
  rc = make_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, (uint32_t)BN);
  if (rc) return 2000 + rc;
  if (BN == 256)
    return mode == MODE_AG ? launch<256, MODE_AG>(ma, mal, mb, mc, dm, p, grid, stream)
                           : launch<256, MODE_RS>(ma, mal, mb, mc, dm, p, grid, stream);
  return mode == MODE_AG ? launch<128, MODE_AG>(ma, mal, mb, mc, dm, p, grid, stream)
                         : launch<128, MODE_RS>(ma, mal, mb, mc, dm, p, grid, stream);
}
