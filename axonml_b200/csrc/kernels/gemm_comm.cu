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
//           Every rank computes its whole partial product tile by tile.  The epilogue sends each
//           finished tile in bf16 (TMEM -> shared memory -> contiguous 4 KB bulk stores, which need
//           no thread while they are in flight) into slot `source rank` of the staging buffer of the
//           rank that owns those rows, its own tiles into its own slot, and raises the tile's flag
//           there one tile later, when the stores have landed.  The accumulator is released as
//           soon as the tile is in shared memory: the math never waits for the network.  All ranks
//           walk the tiles in the same order, so the W copies of a tile exist at about the same time.
//           Reducer warps (four dedicated ones per CTA, joined by the epilogue warps when those
//           run out of tiles) take the tiles of this rank's own rows: when the W flags of a tile
//           are up they add its W staged copies, all in local memory by then, in fp32, add the
//           bias, apply the activation and write the output.  Deterministic (no atomics on data).
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
constexpr int kThreadsRS = 320;    // MODE_RS adds warps 6..9: reducers of this rank's own rows
constexpr int kEpiWarps = 4;
constexpr int kStageBufBytes = 32 * 128;
constexpr int kSigDone = 0;        // [kMaxRanks] "rank p consumed call e"
constexpr int kSigCounter = 8;     // local: CTAs of this rank that finished the call
constexpr int kSigFlags = 16;      // [world][max_tiles][4] chunk / tile flags (RS: one per epilogue warp)
constexpr int kFlagsPerTile = 4;
constexpr int kFlagLag = 3;        // MODE_RS: tiles between a tile's stores and its flag

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
  int fill_own;              // AG: the copy CTAs also fill this rank's own slot of its gathered buffer
  int lazy_done;             // AG: "call e consumed" is sent at the start of call e+1 instead of the end of
                             //     call e, because later kernels on the stream still read the gathered buffer
  int rs_pull;               // RS: partial tiles stay in the sender's staging buffer and the owner of the rows
                             //     adds them up with one multimem load-reduce through the switch
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

// Tile t of the schedule -> (shard, m block inside the shard, n block).  Tiles are taken in groups
// of `g` 128-row blocks of every shard (g * W row blocks, about eight); inside a group the column
// block is the outer index, so CTAs that run together share B tiles and the group's rows of A stay
// in L2 while all column blocks sweep over them.
//  AG: the pushers send block c of every shard at about the same time (one multimem store or one
//      round of bulk stores reaches all peers), so the blocks are consumed in that order; inside a
//      group the ring starts at this rank's own shard, which needs no transfer.
//  RS: the same order on every rank, so that the W partial copies of a tile exist at about the
//      same time and its owner can add them up while the next tiles are computed.
struct TileMap {
  int mbs, num_n, rank, world, rs, g;
  __device__ __forceinline__ void coords(int t, int& shard, int& mb, int& nb) const {
    const int per_group = g * world * num_n;
    const int grp = t / per_group;
    const int first = grp * g;
    const int gsz = min(g, mbs - first);
    const int r = t - grp * per_group;
    const int rows = gsz * world;
    nb = r / rows;
    const int m = r - nb * rows;
    const int pos = m / gsz;
    mb = first + (m - pos * gsz);
    shard = rs ? pos : (rank + pos) % world;
  }
};

// RS staging buffer of a rank: [source rank][128-row block][64-column chunk][row quarter] pieces
// of 4 KB, each the shared-memory image (128-byte swizzle) of a 32 x 64 bf16 sub-tile.
__device__ __forceinline__ long stage_off(int mbs, int N, int src, int mb, int chunk, int quarter) {
  const int nchunks = (N + 63) >> 6;
  return ((((long)src * mbs + mb) * nchunks + chunk) * kEpiWarps + quarter) * (long)kStageBufBytes;
}

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
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    // stream order has put every reader of the previous call's gathered rows on this GPU before this launch
    if (p.lazy_done && pusher == 0) st_release_sys(p.sig[threadIdx.x] + kSigDone + p.rank, p.epoch - 1);
    if (!wait_ge<true>(p.sig[p.rank] + kSigDone + threadIdx.x, p.epoch - 1, p.status, 802)) s_ok = 0;
  }
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
  if (p.lazy_done && pusher == 0) {
    __threadfence_system();
    for (int q = 0; q < p.world; ++q)
      if (q != p.rank) st_release_sys(p.sig[q] + kSigDone + p.rank, p.epoch - 1);
  }
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
    for (int q = p.fill_own ? 0 : 1; q < p.world; ++q)
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
    if (old + 1 == p.epoch * gridDim.x && !p.lazy_done) {
      for (int q = 0; q < p.world; ++q)
        if (q != p.rank) st_release_sys(p.sig[q] + kSigDone + p.rank, p.epoch);
    }
  }
}

// Reduction of this rank's own rows (MODE_RS).  Work items are (own tile of this CTA, row quarter)
// pairs handed out through a shared counter, in tile order.  A warp adds the W staged copies of
// the quarter's 4 KB pieces; lane l owns the 16-byte units l, l + 32, ... of a piece (unit u = row
// u / 8, physical chunk u % 8 of the swizzled image).
template <int BN>
__device__ void reduce_own_rows(const CommParams& p, const TileMap& tm, int cta, int ncta, int* next_item, int lane) {
  const uint32_t* my_flags = p.sig[p.rank] + kSigFlags;
  const int own_tiles = tm.mbs * tm.num_n;
  const int my_tiles = own_tiles > cta ? (own_tiles - cta + ncta - 1) / ncta : 0;
  const uint8_t* stage = p.sym[p.rank];
  while (true) {
    int item = 0;
    if (lane == 0) item = atomicAdd(next_item, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= my_tiles * kEpiWarps) return;
    const int j = cta + (item / kEpiWarps) * ncta;
    const int quarter = item % kEpiWarps;
    const int mb = j / tm.num_n, nb = j - mb * tm.num_n;
    bool w_ok = true;      // lane l: this quarter of the tile as sent by rank l
    if (lane < p.world)
      w_ok = wait_ge<true>(my_flags + ((lane * p.max_tiles + j) * kFlagsPerTile + quarter), p.epoch, p.status, 840);
    if (!__all_sync(0xffffffffu, w_ok)) return;
    __syncwarp();              // the loads below follow the flag reads of the polling lanes
#pragma unroll 1
    for (int ch = 0; ch < BN / 64; ++ch) {
      const int ncol0 = nb * BN + ch * 64;
      if (ncol0 >= p.N) break;
      float a[8][8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) a[i][e] = 0.f;
      if (p.rs_pull) {
        // every rank holds its partial copy of this piece at the same offset of its own buffer:
        // the switch fetches the W copies, adds them in fp32 and returns one
        const uint8_t* piece = p.sym_mc + stage_off(tm.mbs, p.N, p.rank, mb, ncol0 >> 6, quarter) + lane * 16;
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = multimem_ld_reduce_bf16x8(piece + i * 512);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 f0 = unpack_bf16x2(v[i].x), f1 = unpack_bf16x2(v[i].y), f2 = unpack_bf16x2(v[i].z),
                       f3 = unpack_bf16x2(v[i].w);
          a[i][0] = f0.x; a[i][1] = f0.y; a[i][2] = f1.x; a[i][3] = f1.y;
          a[i][4] = f2.x; a[i][5] = f2.y; a[i][6] = f3.x; a[i][7] = f3.y;
        }
      }
      for (int src = 0; src < (p.rs_pull ? 0 : p.world); ++src) {
        const uint8_t* piece = stage + stage_off(tm.mbs, p.N, src, mb, ncol0 >> 6, quarter) + lane * 16;
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = ld_peer_v4(piece + i * 512);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 f0 = unpack_bf16x2(v[i].x), f1 = unpack_bf16x2(v[i].y), f2 = unpack_bf16x2(v[i].z),
                       f3 = unpack_bf16x2(v[i].w);
          a[i][0] += f0.x; a[i][1] += f0.y; a[i][2] += f1.x; a[i][3] += f1.y;
          a[i][4] += f2.x; a[i][5] += f2.y; a[i][6] += f3.x; a[i][7] += f3.y;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int u = lane + 32 * i;
        const int row = u >> 3;
        const int col = ncol0 + (((u & 7) ^ (row & 7)) << 3);      // logical 8-column group of this unit
        if (p.bias_kind == 1) {
#pragma unroll
          for (int e = 0; e < 8; ++e) a[i][e] += __ldg((const float*)p.bias + col + e);
        } else if (p.bias_kind == 2) {
#pragma unroll
          for (int e = 0; e < 8; ++e) a[i][e] += __bfloat162float(((const __nv_bfloat16*)p.bias)[col + e]);
        }
        if (p.act != kActNone) {
#pragma unroll
          for (int e = 0; e < 8; ++e) a[i][e] = apply_act(a[i][e], p.act);
        }
        uint4 o;
        o.x = pack_bf16x2(a[i][0], a[i][1]); o.y = pack_bf16x2(a[i][2], a[i][3]);
        o.z = pack_bf16x2(a[i][4], a[i][5]); o.w = pack_bf16x2(a[i][6], a[i][7]);
        *reinterpret_cast<uint4*>(p.out + (((long)(mb * BM + quarter * 32 + row)) * p.N + col) * 2) = o;
      }
    }
  }
}

template <int BN, int MODE, int B_MN>
__global__ void __launch_bounds__(MODE == MODE_RS ? kThreadsRS : kThreads, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_local,
                 const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                 const CommParams p) {
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
  tm.rs = MODE == MODE_RS ? 1 : 0;
  tm.g = max(1, 8 / p.world);
  __shared__ int s_next_item;
  const int num_tiles = p.world * tm.mbs * tm.num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  uint32_t* my_flags = p.sig[p.rank] + kSigFlags;

  if (threadIdx.x == 0) {
    trace_at(p, 0);
    *dead = 0;
    s_next_item = 0;
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
        int shard, mb, nb;
        tm.coords(t, shard, mb, nb);
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
          uint8_t* sb = sa + C::kStageA;
          mbar_expect_tx(&full_bar[s], C::kStage);
          tma_load_2d(sa, ma, &full_bar[s], kb * BK, m0);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &map_b, &full_bar[s], n0 + j * 64, kb * BK);
          } else {
            tma_load_2d(sb, &map_b, &full_bar[s], kb * BK, n0);
          }
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        if (*dead) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(1, BM, BN, 0, B_MN);
      // descriptors of stage 0, advanced per stage and k step (keeps the issuing thread short)
      const uint64_t da0 = umma_desc_sw128(smem_u32(stage_base), 16, 1024);
      const uint64_t db0 = B_MN ? umma_desc_sw128(smem_u32(stage_base) + C::kStageA, BK * 128, 1024)
                                : umma_desc_sw128(smem_u32(stage_base) + C::kStageA, 16, 1024);
      constexpr uint32_t kStepA = (UMMA_K * 2) >> 4;
      constexpr uint32_t kStepB = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
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
            umma_f16_ss(d_tmem, da0 + soff + (uint64_t)(k * kStepA), db0 + soff + (uint64_t)(k * kStepB),
                        idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        umma_commit(&tfull_bar[acc]);
        if (it < 15) trace_at(p, 2 + 4 * it + 3);
        if (*dead) break;
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;            // TMEM lane quarter = row quarter of the tile this warp drains
    const int ew = warp - 2;
    uint8_t* stg = epi_base + ew * 2 * kStageBufBytes;
    int buf = 0, it = 0;
    // The tiles whose flags are still owed.  The flag of a tile goes out kFlagLag tiles
    // later: a completion wait right after the stores costs a full trip through the switch, which
    // under the all-to-all load of eight ranks is tens of microseconds.
    int pend_shard[kFlagLag], pend_tile[kFlagLag];
#pragma unroll
    for (int i = 0; i < kFlagLag; ++i) { pend_shard[i] = -1; pend_tile[i] = 0; }
    bool ok = true;
    if (MODE == MODE_RS) {
      // the peers must have added up the previous call's partial tiles before their staging slots
      // are overwritten (every warp checks for itself: no barrier that a timed-out warp could
      // leave hanging)
      bool w_ok = true;
      if (lane < p.world && lane != p.rank) w_ok = wait_ge<true>(p.sig[p.rank] + kSigDone + lane, p.epoch - 1, p.status, 830);
      ok = __all_sync(0xffffffffu, w_ok);
      if (!ok) *dead = 1;      // the producer and MMA warps stop at their next wait
    }
    if (ew == 0 && lane == 0) trace_at(p, 1);
    for (int t = cta; t < num_tiles && ok; t += ncta, ++it) {
      int shard, mb, nb;
      tm.coords(t, shard, mb, nb);
      const int m0 = shard * p.Tl + mb * BM, n0 = nb * BN;
      const int acc = it & 1;
      ok = mbar_wait(&tfull_bar[acc], (it >> 1) & 1, dead, p.status, 831);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (ew == 0 && lane == 0 && it < 15) trace_at(p, 2 + 4 * it);
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
        if (ncol0 >= p.N) {
          // every tile commits BN / 64 store groups, empty ones included: the flag logic below counts them
          if (MODE == MODE_RS && lane == 0) tma_store_commit();
          continue;
        }
        if (MODE == MODE_AG) {
          add_bias_chunk(r, p.bias, p.bias_kind, ncol0, p.N);
          apply_act_chunk(r, p.act);
        }
        // AG: a tile of the result (tensor store).  RS: a partial tile for the owner of these rows,
        // sent as one contiguous 4 KB piece per warp and chunk (row-strided 128-byte writes over
        // NVLink ran at a third of the rate); this rank's own tiles take the same path locally.
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
          if (MODE == MODE_AG) tma_store_2d(&map_c, dst, ncol0, m0 + q * 32);
          else if (p.rs_pull) bulk_store_1d(p.sym[p.rank] + stage_off(tm.mbs, p.N, shard, mb, ncol0 >> 6, q), dst, kStageBufBytes);
          else bulk_store_1d(p.sym[shard] + stage_off(tm.mbs, p.N, p.rank, mb, ncol0 >> 6, q), dst, kStageBufBytes);
          tma_store_commit();
        }
        buf ^= 1;
      }
      if (MODE == MODE_RS) {
        if (ew == 0 && lane == 0 && it < 15) trace_at(p, 2 + 4 * it + 1);
        // Lane 0 issued the stores, so only it can wait for them; the flag is raised by lane 1.  A
        // system-scope fence or release by lane 0 would also wait for the stores of the later tiles it
        // has in flight (22 us per tile on four GPUs), which is what the lag is there to avoid; lane 1
        // has no writes of its own, and its release is ordered after lane 0's wait by the warp barrier.
        if (pend_shard[0] >= 0) {
          if (lane == 0) {
            tma_store_wait<kFlagLag * (BN / 64)>();      // everything but the stores of the last kFlagLag tiles
            fence_proxy_async_global();
          }
          __syncwarp();
          if (lane == 1)
            st_release_sys(p.sig[pend_shard[0]] + kSigFlags + ((p.rank * p.max_tiles + pend_tile[0]) * kFlagsPerTile + q), p.epoch);
        }
#pragma unroll
        for (int i = 0; i + 1 < kFlagLag; ++i) { pend_shard[i] = pend_shard[i + 1]; pend_tile[i] = pend_tile[i + 1]; }
        pend_shard[kFlagLag - 1] = shard;
        pend_tile[kFlagLag - 1] = mb * tm.num_n + nb;
        __syncwarp();
      }
      if (ew == 0 && lane == 0 && it < 15) trace_at(p, 2 + 4 * it + 2);
    }
    __syncwarp();
    if (ew == 0 && lane == 0) trace_at(p, 62);
    if (lane == 0) {
      tma_store_wait<0>();
      if (MODE == MODE_RS) fence_proxy_async_global();
    }
    __syncwarp();
    if (MODE == MODE_RS && lane == 1) {
#pragma unroll
      for (int i = 0; i < kFlagLag; ++i)
        if (pend_shard[i] >= 0)
          st_release_sys(p.sig[pend_shard[i]] + kSigFlags + ((p.rank * p.max_tiles + pend_tile[i]) * kFlagsPerTile + q), p.epoch);
    }
    __syncwarp();
    // out of tiles: help with the reduction of this rank's own rows
    if (MODE == MODE_RS && ok) reduce_own_rows<BN>(p, tm, cta, ncta, &s_next_item, lane);
  } else if (MODE == MODE_RS) {
    // ------------------------------------------------------------ reducers of this rank's rows
    reduce_own_rows<BN>(p, tm, cta, ncta, &s_next_item, lane);
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

template <int BN, int MODE, int B_MN>
int launch(const CUtensorMap& ma, const CUtensorMap& mal, const CUtensorMap& mb, const CUtensorMap& mc,
           const CommParams& p, int grid, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_comm_kernel<BN, MODE, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, MODE == MODE_RS ? kThreadsRS : kThreads, C::kSmem, stream>>>(ma, mal, mb, mc, p);
  return (int)cudaGetLastError();
}

template <int BN, int MODE>
int launch_b(int b_mn, const CUtensorMap& ma, const CUtensorMap& mal, const CUtensorMap& mb, const CUtensorMap& mc,
             const CommParams& p, int grid, cudaStream_t stream) {
  return b_mn ? launch<BN, MODE, 1>(ma, mal, mb, mc, p, grid, stream) : launch<BN, MODE, 0>(ma, mal, mb, mc, p, grid, stream);
}

}  // namespace

// Number of 32-bit slots a communicator's signal array needs for `max_tiles` flags per rank.
AX_API int ax_gemm_comm_signal_slots(int max_tiles) { return kSigFlags + kMaxRanks * max_tiles * kFlagsPerTile; }

// Diagnostic timeline: the launches that follow write globaltimer stamps of their phases into
// `buf` ([grid][64] 64-bit slots, zero-filled by the caller); null turns it off again.
static unsigned long long* g_trace_buf = nullptr;
static int g_rs_pull = -1;
AX_API void ax_gemm_comm_set_trace(void* buf) { g_trace_buf = (unsigned long long*)buf; }

// mode 0: C[world*Tl, N] = act(allgather(x_local)[world*Tl, K] * op(B) + bias); `sym` = gathered buffers
//         [world][Tl][K], `out` = C (row stride N).
// mode 1: out[Tl, N] = act(reduce_scatter(x[world*Tl, K] * op(B)) + bias); `sym` = staging buffers
//         (world * Tl * N bf16 each, one slot per source rank), `x_local` = x.
//         With `keep_gathered` every rank's gathered buffer is complete (own rows included) when the
//         launch has finished and stays valid until the next call on this communicator, for later
//         kernels on the same stream (the weight gradient of the layer); all calls on one communicator
//         must then use keep_gathered.
// op(B): b_mn = 0: B is [N, K] row-major (a Linear weight); b_mn = 1: B is [K, N] row-major.
// `grid` must be the same for every call on one communicator (the end-of-call counter relies on it)
// and must not exceed the SM count.  Requires Tl % 128 == 0, K % 64 == 0, N % 64 == 0.
// Reduce-scatter transport of MODE_RS: -1 = by rank count (in-switch reduction above two ranks when a
// multicast mapping exists), 0 = partial tiles are pushed to the owner, 1 = the owner pulls the sum.
AX_API void ax_gemm_comm_set_rs_pull(int mode) { g_rs_pull = mode; }

AX_API int ax_gemm_comm(int mode, const void* x_local, const void* B, void* out, void* const* sym, void* sym_mc,
                        void* const* sig, const void* bias, int bias_kind, int act, int Tl, int N, int K,
                        int b_mn, int rank, int world, unsigned epoch, int max_tiles, int pushers, int grid,
                        int keep_gathered, int* status, cudaStream_t stream) {
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
  p.fill_own = p.lazy_done = (mode == MODE_AG && keep_gathered) ? 1 : 0;
  // reduce-scatter transport: the in-switch reduction needs the multicast mapping; with two ranks the
  // switch has nothing to add up and the push form (no read round trip) is faster
  p.rs_pull = (mode == MODE_RS && sym_mc != nullptr && (g_rs_pull == 1 || (g_rs_pull < 0 && world > 2))) ? 1 : 0;
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
    mc = ma;        // not used: partial tiles leave as plain bulk stores, the reducers write `out` directly
  }
  if (b_mn) rc = make_map_2d(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)N, 64, BK);
  else rc = make_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, (uint32_t)BN);
  if (rc) return 2000 + rc;
  if (BN == 256)
    return mode == MODE_AG ? launch_b<256, MODE_AG>(b_mn, ma, mal, mb, mc, p, grid, stream)
                           : launch_b<256, MODE_RS>(b_mn, ma, mal, mb, mc, p, grid, stream);
  return mode == MODE_AG ? launch_b<128, MODE_AG>(b_mn, ma, mal, mb, mc, p, grid, stream)
                         : launch_b<128, MODE_RS>(b_mn, ma, mal, mb, mc, p, grid, stream);
}
