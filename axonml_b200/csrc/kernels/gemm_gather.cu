// FSDP parameter all-gather fused into the first GEMM that consumes the parameters:
//
//   C[M, N] = act(X[M, K] * W[N, K]^T + bias),   W = rows of a flat parameter buffer that is sharded
//                                                 over the ranks and gathered by this same launch.
//
// A sharded unit keeps its parameters back to back in one flat bf16 buffer of `total` elements;
// rank r owns elements [r * shard, (r + 1) * shard) (its up-to-date "shard") and every rank has a
// full-size buffer in symmetric memory that the parameters view.  One launch does both jobs:
//
//  * a few CTA pairs only copy: they send this rank's shard, 64 KB chunk after chunk, into the same
//    place of every rank's full buffer, its own included (bulk loads into shared memory, then one
//    NVSwitch multimem store per 16 bytes, or bulk stores to each peer when no multicast mapping
//    exists), and raise the chunk's flag on every rank when the chunk has landed;
//  * the other CTA pairs run the CTA-pair GEMM of gemm_tcgen05.cu (tcgen05 cta_group::2, 256 x 256
//    tiles, plain TMA loads of this GPU's own memory).  Their TMA producer waits, before the first
//    load of a tile, for the flags of the chunks that hold the tile's rows of W.  Tiles are taken
//    column block by column block, the order in which W's rows arrive, so the math starts as soon as
//    the first chunks are there and the transfer overlaps it.
//
// The launch ends only when every chunk of the unit has arrived on this rank (one copy CTA checks
// all flags), so the unit's other layers, which run as later kernels on the same stream, read a
// complete buffer.  A rank tells its peers at the start of a launch that the previous contents of
// its buffer are no longer read (everything that read them precedes this launch on the stream);
// nobody writes a peer's buffer before that.  Flags hold the launch's epoch and only grow; every
// wait is bounded and reports through the status word.
//
// Replaces gather_parameters (crates/axonml-distributed/src/fsdp.rs:215-235: an all_gather per
// parameter on a mock backend) followed by the Linear forward
// (crates/axonml-nn/src/layers/linear.rs:104-140).
#include "comm.cuh"

namespace {
using namespace ax;
using namespace axc;

constexpr int BM = 128;            // rows per CTA (256 per pair)
constexpr int BN = 256;            // columns per pair tile (128 rows of W per CTA)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
constexpr int kStageBufBytes = 32 * 128;
constexpr int kStageA = BM * BK * 2;
constexpr int kStageB = (BN / 2) * BK * 2;
constexpr int kStage = kStageA + kStageB;
constexpr int kStages = 6;
constexpr int kSmem = 1024 + kStages * kStage + kEpiWarps * 2 * kStageBufBytes + 256;
constexpr int kChunkElems = 32768;                 // 64 KB of bf16: the unit of arrival
constexpr int kPiece = 16384;                      // bytes per bulk copy
constexpr int kPieces = 12;                        // pieces in flight per copy CTA (192 KB)
constexpr int kSigDone = 0;                        // [kMaxRanks] "rank p no longer reads epoch e - 1"
constexpr int kSigFlags = 16;                      // [world * chunks_per_shard] chunk flags

struct GatherParams {
  int M, N, K;
  long w_off;                 // element offset of W inside the flat buffer
  long shard, total;          // elements per rank, elements in the flat buffer
  int chunks_per_shard;
  int rank, world;
  uint32_t epoch;
  uint32_t* sig[kMaxRanks];
  uint8_t* full[kMaxRanks];   // every rank's full buffer (peer-mapped)
  uint8_t* full_mc;           // multicast mapping of the full buffers, or null
  const uint8_t* shard_src;   // this rank's shard (shard * 2 bytes)
  const void* bias;
  int bias_kind, act;
  int copy_pairs;             // CTA pairs that only copy
  int* status;
};

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
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// Copy CTA `me` of `n`: chunks me, me + n, ... of this rank's shard go to every rank's full buffer.
__device__ void copy_shard(const GatherParams& p, int me, int n, uint8_t* smem) {
  uint8_t* buf = smem;                                             // [kPieces][kPiece]
  uint64_t* full = (uint64_t*)(smem + kPieces * kPiece);           // [kPieces]
  volatile int* dead = (volatile int*)(full + kPieces);
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_ok = 1;
    *dead = 0;
    for (int i = 0; i < kPieces; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    // every reader of the buffer's previous contents on this GPU precedes this launch on its stream
    if (me == 0) {
      __threadfence_system();
      st_release_sys(p.sig[threadIdx.x] + kSigDone + p.rank, p.epoch - 1);
    }
    if (!wait_ge<true>(p.sig[p.rank] + kSigDone + threadIdx.x, p.epoch - 1, p.status, 900)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const long shard_bytes = p.shard * 2;
  const long chunk_bytes = (long)kChunkElems * 2;
  // pieces of my chunks, in order
  long total = 0;
  for (int c = me; c < p.chunks_per_shard; c += n) {
    const long cb = min(chunk_bytes, shard_bytes - (long)c * chunk_bytes);
    total += (cb + kPiece - 1) / kPiece;
  }
  const bool mc = p.full_mc != nullptr && p.world > 2;
  // iterate pieces with a small cursor: (chunk, piece inside the chunk)
  struct Cursor { int c; int k; };
  auto advance = [&](Cursor& cu) {
    const long cb = min(chunk_bytes, shard_bytes - (long)cu.c * chunk_bytes);
    if ((long)(cu.k + 1) * kPiece < cb) ++cu.k; else { cu.c += n; cu.k = 0; }
  };
  auto piece_bytes = [&](const Cursor& cu) -> uint32_t {
    const long cb = min(chunk_bytes, shard_bytes - (long)cu.c * chunk_bytes);
    return (uint32_t)min((long)kPiece, cb - (long)cu.k * kPiece);
  };
  auto piece_off = [&](const Cursor& cu) -> long { return (long)cu.c * chunk_bytes + (long)cu.k * kPiece; };
  Cursor ld{me, 0}, cur{me, 0};
  long issued = 0;
  if (threadIdx.x == 0) {
    for (; issued < kPieces - 2 && issued < total; ++issued) {
      const uint32_t b = piece_bytes(ld);
      mbar_expect_tx(&full[issued % kPieces], b);
      bulk_load_1d(buf + (issued % kPieces) * kPiece, p.shard_src + piece_off(ld), b, &full[issued % kPieces]);
      advance(ld);
    }
  }
  for (long i = 0; i < total; ++i) {
    const int st = (int)(i % kPieces);
    if (threadIdx.x == 0 && issued < total) {
      // piece `issued` takes the stage of piece i - 2, whose stores had been read (or whose
      // multimem copies had been issued) when round i - 1 ended
      const uint32_t b = piece_bytes(ld);
      mbar_expect_tx(&full[issued % kPieces], b);
      bulk_load_1d(buf + (issued % kPieces) * kPiece, p.shard_src + piece_off(ld), b, &full[issued % kPieces]);
      advance(ld);
      ++issued;
    }
    const bool ok = mbar_wait(&full[st], (uint32_t)((i / kPieces) & 1), dead, p.status, 901);
    if (!__syncthreads_and(ok)) return;
    const uint32_t bytes = piece_bytes(cur);
    const long dst_off = (long)p.rank * shard_bytes + piece_off(cur);
    if (mc) {
      const uint32_t sbase = smem_u32(buf + st * kPiece);
      for (int j = threadIdx.x; j < (int)(bytes / 16); j += kThreads) {
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(sbase + j * 16));
        multimem_st_b32x4(p.full_mc + dst_off + (long)j * 16, v);
      }
    } else if (threadIdx.x == 0) {
      for (int q = 0; q < p.world; ++q)
        bulk_store_1d(p.full[(p.rank + q) % p.world] + dst_off, buf + st * kPiece, bytes);
      tma_store_commit();
    }
    const long cb = min(chunk_bytes, shard_bytes - (long)cur.c * chunk_bytes);
    const bool chunk_done = (long)(cur.k + 1) * kPiece >= cb;
    if (chunk_done) {
      if (!mc && threadIdx.x == 0) {
        tma_store_wait<0>();             // the chunk has landed everywhere
        fence_proxy_async_global();
      }
      __threadfence_system();
    } else if (!mc && threadIdx.x == 0) {
      tma_store_wait_read<1>();            // all but the latest group of stores have read their stage
    }
    __syncthreads();
    if (chunk_done && (int)threadIdx.x < p.world)
      st_release_sys(p.sig[threadIdx.x] + kSigFlags + p.rank * p.chunks_per_shard + cur.c, p.epoch);
    advance(cur);
  }
  if (!mc && threadIdx.x == 0) tma_store_wait<0>();
}

// All chunks of all ranks have arrived here (one CTA checks on behalf of the launch).
__device__ void wait_all_chunks(const GatherParams& p) {
  const uint32_t* flags = p.sig[p.rank] + kSigFlags;
  const int n = p.world * p.chunks_per_shard;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    if (!wait_ge<true>(flags + i, p.epoch, p.status, 902)) return;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_gather_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_c, const GatherParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t crank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  if (pair_id < p.copy_pairs) {
    // both CTAs of a copy pair copy; neither touches the other's shared memory, so no cluster sync
    copy_shard(p, (int)blockIdx.x, 2 * p.copy_pairs, smem);
    __syncthreads();
    if (blockIdx.x == 0) wait_all_chunks(p);
    return;
  }
  uint8_t* stage_base = smem;
  uint8_t* epi_base = smem + kStages * kStage;
  uint64_t* bars = (uint64_t*)(epi_base + kEpiWarps * 2 * kStageBufBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tfull_bar = bars + 2 * kStages;
  uint64_t* tempty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 4);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cpair = pair_id - p.copy_pairs;
  const int npairs = (gridDim.x >> 1) - p.copy_pairs;
  constexpr int PM = 2 * BM, HB = BN / 2;
  const int num_m = (p.M + PM - 1) / PM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 2 * kEpiWarps); }
    mbar_fence_init();
    prefetch_tensormap(&map_a); prefetch_tensormap(&map_b); prefetch_tensormap(&map_c);
  }
  if (warp == 1) { tmem_alloc_pair<512>(tmem_slot); tmem_relinquish_pair(); }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // column block outermost: the order in which the rows of W arrive
  auto tile_coords = [&](int t, int& mb, int& nb) { nb = t / num_m; mb = t - nb * num_m; };

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t* flags = p.sig[p.rank] + kSigFlags;
      int s = 0;
      uint32_t ph = 0;
      int ready_nb = -1;                         // column block whose rows this CTA has seen arrive
      for (int t = cpair; t < num_tiles; t += npairs) {
        int mb, nb;
        tile_coords(t, mb, nb);
        const int m0 = mb * PM + (int)crank * BM, n0 = nb * BN + (int)crank * HB;
        if (nb != ready_nb) {
          // rows [n0, n0 + HB) of W = flat elements [w_off + n0 K, w_off + min(n0 + HB, N) K)
          const int rows_end = min(n0 + HB, p.N);
          bool ok = true;
          if (n0 < rows_end) {
            const long e0 = p.w_off + (long)n0 * p.K, e1 = p.w_off + (long)rows_end * p.K - 1;
            for (long e = e0; ok;) {
              const int src = (int)(e / p.shard);
              const int c = (int)((e - (long)src * p.shard) / kChunkElems);
              ok = wait_ge<true>(flags + src * p.chunks_per_shard + c, p.epoch, p.status, 910);
              const long next = (long)src * p.shard + min((long)(c + 1) * kChunkElems, p.shard);   // first element of the next chunk
              if (next > e1) break;
              e = next;
            }
          }
          if (!ok) { *dead = 1; break; }
          fence_proxy_async_global();            // the peers' writes before this CTA's TMA reads
          ready_nb = nb;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 911)) break;
          uint8_t* sa = stage_base + s * kStage;
          if (crank == 0) mbar_expect_tx(&full_bar[s], 2 * kStage);
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[s]), 0);
          tma_load_2d_pair(sa, &map_a, fb, kb * BK, m0);
          tma_load_2d_pair(sa + kStageA, &map_b, fb, kb * BK, n0);
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (*dead) break;
      }
      for (int i = 0; i < kStages && !*dead; ++i) {
        if (!mbar_wait(&empty_bar[s], ph ^ 1, dead, p.status, 912)) break;
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && crank == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(1, PM, BN, 0, 0);
      const uint32_t sa0 = smem_u32(stage_base);
      const uint64_t da0 = umma_desc_sw128(sa0, 16, 1024);
      const uint64_t db0 = umma_desc_sw128(sa0 + kStageA, 16, 1024);
      int s = 0, it = 0;
      uint32_t ph = 0;
      for (int t = cpair; t < num_tiles; t += npairs, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, dead, p.status, 920)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, dead, p.status, 921)) break;
          tc_fence_after();
          const uint64_t soff = (uint64_t)((uint32_t)(s * kStage) >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_ss_pair(d_tmem, da0 + soff + (uint64_t)(k * 2), db0 + soff + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty_bar[s]);
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        umma_commit_pair(&tfull_bar[acc]);
        if (*dead) break;
      }
    }
  } else {
    const int q = warp & 3, ew = warp - 2;
    uint8_t* stg = epi_base + ew * 2 * kStageBufBytes;
    const uint32_t tempty_leader0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    int buf = 0, it = 0;
    for (int t = cpair; t < num_tiles; t += npairs, ++it) {
      int mb, nb;
      tile_coords(t, mb, nb);
      const int m0 = mb * PM + (int)crank * BM, n0 = nb * BN;
      const int acc = it & 1;
      bool ok = mbar_wait(&tfull_bar[acc], (it >> 1) & 1, dead, p.status, 930);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int ch = 0; ch < BN / 64; ++ch) {
        uint32_t r[64];
        tmem_ld_32x32b_x32(t_row + ch * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld_32x32b_x32(t_row + ch * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tc_wait_ld();
        if (ch == BN / 64 - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_leader0 + acc * 8);
        }
        const int ncol0 = n0 + ch * 64;
        if (ncol0 >= p.N || m0 + q * 32 >= p.M) continue;
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
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair<512>(tmem_base);
}

int make_map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {ld_elems * 2};
  uint32_t box[2] = {box_inner, box_outer};
  return axh::encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

// 32-bit signal slots a unit's communicator needs for a flat buffer of `total` elements over `world` ranks.
AX_API int ax_gemm_gather_signal_slots(long total, int world) {
  const long shard = total / world;
  return kSigFlags + world * (int)((shard + kChunkElems - 1) / kChunkElems);
}

// Gathers the flat parameter buffer (`shard_src`: this rank's shard of `total / world` elements ->
// element offset rank * shard of every rank's `full[...]`) and computes
// C[M, N] = act(X[M, K] * W^T + bias) with W = [N, K] at element offset `w_off` of this rank's full
// buffer, in one launch.  `epoch` grows by one per launch on these buffers and signals (the same
// on every rank).  `copy_pairs` CTA pairs only copy; the grid is as many pairs as the device runs
// at once.  Requires K % 64 == 0, N % 8 == 0, w_off % 8 == 0, total % (64 * world) == 0.
// Returns a cudaError_t value, -1 for a bad argument, -3 when CTA pairs cannot be launched.
AX_API int ax_gemm_gather(const void* X, void* C, const void* bias, int bias_kind, int act, int M, int N, int K,
                          long w_off, long total, const void* shard_src, void* const* full, void* full_mc,
                          void* const* sig, int rank, int world, unsigned epoch, int copy_pairs, int* status,
                          cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || M <= 0 || N <= 0 || K <= 0 || K % BK || N % 8 || w_off % 8) return -1;
  if (total % (64L * world) || w_off + (long)N * K > total || copy_pairs < 1) return -1;
  GatherParams p;
  p.M = M; p.N = N; p.K = K; p.w_off = w_off; p.total = total; p.shard = total / world;
  p.chunks_per_shard = (int)((p.shard + kChunkElems - 1) / kChunkElems);
  p.rank = rank; p.world = world; p.epoch = epoch;
  for (int i = 0; i < kMaxRanks; ++i) {
    p.sig[i] = i < world ? (uint32_t*)sig[i] : nullptr;
    p.full[i] = i < world ? (uint8_t*)full[i] : nullptr;
  }
  p.full_mc = (uint8_t*)full_mc;
  p.shard_src = (const uint8_t*)shard_src;
  p.bias = bias; p.bias_kind = bias ? bias_kind : 0; p.act = act;
  p.status = status;
  CUtensorMap ma, mb, mc;
  int rc;
  if ((rc = make_map_2d(&ma, X, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, BM))) return 1000 + rc;
  if ((rc = make_map_2d(&mb, (const uint8_t*)full[rank] + w_off * 2, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, BN / 2))) return 2000 + rc;
  if ((rc = make_map_2d(&mc, C, (uint64_t)N, (uint64_t)M, (uint64_t)N, 64, 32))) return 3000 + rc;

  static int max_pairs[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs[dev] == 0) {
    cudaError_t e = cudaFuncSetAttribute(gemm_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return (int)e;
    cfg.gridDim = dim3(2 * axh::sm_count(), 1, 1);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, (const void*)gemm_gather_kernel, &cfg);
    if (e != cudaSuccess) return (int)e;
    if (n < 2) return -3;
    max_pairs[dev] = n;
  }
  // every pair must be resident: the copy pairs and the math pairs wait for one another's work
  int pairs = max_pairs[dev];
  if (copy_pairs >= pairs) copy_pairs = pairs - 1;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  if (pairs > copy_pairs + tiles) pairs = copy_pairs + tiles;
  p.copy_pairs = copy_pairs;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  return (int)cudaLaunchKernelEx(&cfg, gemm_gather_kernel, ma, mb, mc, p);
}
