// Tensor-parallel GEMMs fused with their collective, one launch each, over NVLink peer memory:
//
//  MODE_AG  all-gather -> GEMM (column-parallel Linear with sequence-parallel input):
//           C[W*Tl, N] = act(concat_r(X_r)[W*Tl, K] * B[N, K]^T + bias).
//           A few "pusher" CTAs copy this rank's shard X_rank, 128 rows at a time, into slot `rank`
//           of every peer's gathered buffer (one NVSwitch multimem store per 16 bytes when a
//           multicast mapping exists, else one peer store per peer) and raise a per-chunk flag in
//           the peer's memory.  The GEMM CTAs start on the local shard at once and take the other
//           shards in ring order; the TMA producer of a tile waits for the flag of the chunk it
//           is about to read, so the transfer overlaps the math chunk by chunk.  TMA reads only
//           this GPU's own memory.
//
//  MODE_RS  GEMM -> reduce-scatter (row-parallel Linear with sequence-parallel output):
//           out[Tl, N] = act(sum_r (X_r[W*Tl, Kl] * B_r[N, Kl]^T)[rows of this rank] + bias).
//           Every rank computes its partial product tile by tile, the destination shard after
//           its own first and its own shard last, and the epilogue stores each finished tile
//           (bf16) straight from TMEM into the destination rank's staging slot for this source,
//           then raises a per-tile flag there.  When a CTA has finished its GEMM tiles it reduces
//           tiles of the local shard: waits for the W flags of a tile, sums the W staged copies
//           in fp32 and writes the result.  Deterministic (no floating-point atomics).
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
};

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
__device__ void push_shard(const CommParams& p, int pusher, int npushers) {
  const int chunks = p.Tl / BM;
  const long row_bytes = (long)p.K * 2;
  const long chunk_bytes = (long)BM * row_bytes;
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // the peers must have finished reading what the previous call put there
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank)
    if (!wait_ge<true>(p.sig[p.rank] + kSigDone + threadIdx.x, p.epoch - 1, p.status, 800)) s_ok = 0;
  __syncthreads();
  if (!s_ok) return;
  for (int c = pusher; c < chunks; c += npushers) {
    const uint8_t* src = p.x_local + (long)c * chunk_bytes;
    const long dst_off = ((long)p.rank * p.Tl + (long)c * BM) * row_bytes;
    for (long o = (long)threadIdx.x * 16; o < chunk_bytes; o += (long)blockDim.x * 16) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + o);
      if (p.sym_mc != nullptr) {
        multimem_st_b32x4(p.sym_mc + dst_off + o, v);
      } else {
        for (int q = 1; q < p.world; ++q) st_peer_v4(p.sym[(p.rank + q) % p.world] + dst_off + o, v);
      }
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank)
      st_release_sys(p.sig[threadIdx.x] + kSigFlags + (p.rank * p.max_tiles + c) * kFlagsPerTile, p.epoch);
  }
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

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_local,
                 const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                 const CommParams p) {
  using C = Cfg<BN>;
  if (MODE == MODE_AG && (int)blockIdx.x < p.pushers) {
    push_shard(p, blockIdx.x, p.pushers);
    finish_call(p);
    return;
  }
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
          const uint32_t sa = smem_u32(stage_base + s * C::kStage);
          const uint32_t sb = sa + C::kStageA;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_ss(d_tmem, umma_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024),
                        umma_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
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
    const int et = ew * 32 + lane;            // 0..127 inside the epilogue group
    uint8_t* stg = epi_base + ew * 2 * kStageBufBytes;
    int buf = 0, it = 0;
    bool ok = true;
    if (MODE == MODE_RS) {
      // peers must have consumed the previous call before their staging slots are overwritten
      // (every warp checks for itself: no barrier that a timed-out warp could leave hanging)
      bool w_ok = true;
      if (lane < p.world && lane != p.rank) w_ok = wait_ge<true>(p.sig[p.rank] + kSigDone + lane, p.epoch - 1, p.status, 830);
      ok = __all_sync(0xffffffffu, w_ok);
      if (!ok) *dead = 1;      // the producer and MMA warps stop at their next wait
    }
    for (int t = cta; t < num_tiles && ok; t += ncta, ++it) {
      int ring_pos, shard, mb, nb;
      tm.coords(t, ring_pos, shard, mb, nb);
      const int m0 = shard * p.Tl + mb * BM, n0 = nb * BN;
      const int acc = it & 1;
      ok = mbar_wait(&tfull_bar[acc], (it >> 1) & 1, dead, p.status, 831);
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
        const int ncol0 = n0 + ch * 64;
        if (ncol0 >= p.N) continue;
        if (MODE == MODE_AG) {
          if (p.bias_kind != 0) {
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              const int n = ncol0 + j;
              float b = 0.f;
              if (n < p.N)
                b = p.bias_kind == 1 ? __ldg((const float*)p.bias + n) : __bfloat162float(((const __nv_bfloat16*)p.bias)[n]);
              r[j] = __float_as_uint(__uint_as_float(r[j]) + b);
            }
          }
          uint8_t* dst = stg + buf * kStageBufBytes;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 o;
            o.x = pack_bf16x2(apply_act(__uint_as_float(r[c * 8 + 0]), p.act), apply_act(__uint_as_float(r[c * 8 + 1]), p.act));
            o.y = pack_bf16x2(apply_act(__uint_as_float(r[c * 8 + 2]), p.act), apply_act(__uint_as_float(r[c * 8 + 3]), p.act));
            o.z = pack_bf16x2(apply_act(__uint_as_float(r[c * 8 + 4]), p.act), apply_act(__uint_as_float(r[c * 8 + 5]), p.act));
            o.w = pack_bf16x2(apply_act(__uint_as_float(r[c * 8 + 6]), p.act), apply_act(__uint_as_float(r[c * 8 + 7]), p.act));
            *reinterpret_cast<uint4*>(dst + lane * 128 + ((c ^ (lane & 7)) << 4)) = o;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&map_c, dst, ncol0, m0 + q * 32);
            tma_store_commit();
          }
          buf ^= 1;
        } else {
          // partial tile -> staging slot `rank` on the rank that owns these rows
          uint8_t* dst = p.sym[shard] + (((long)p.rank * p.Tl + mb * BM + q * 32 + lane) * p.N + ncol0) * 2;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[c * 8 + 0]), __uint_as_float(r[c * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[c * 8 + 2]), __uint_as_float(r[c * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[c * 8 + 4]), __uint_as_float(r[c * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[c * 8 + 6]), __uint_as_float(r[c * 8 + 7]));
            if (ncol0 + c * 8 < p.N) st_peer_v4(dst + c * 16, o);
          }
        }
      }
      if (MODE == MODE_RS) {
        // this warp's quarter of the tile is on its way: one flag per epilogue warp
        __threadfence_system();
        __syncwarp();
        if (lane == 0)
          st_release_sys(p.sig[shard] + kSigFlags + ((p.rank * p.max_tiles + mb * tm.num_n + nb) * kFlagsPerTile + ew), p.epoch);
      }
    }
    if (MODE == MODE_AG) {
      if (lane == 0) tma_store_wait<0>();
    } else if (ok) {
      // -------------------------------------------------------- reduce the local shard's tiles
      const int work = tm.mbs * tm.num_n;
      const long row_bytes = (long)p.N * 2;
      for (int w = cta; w < work && ok; w += ncta) {
        const int mb = w / tm.num_n, nb = w - mb * tm.num_n;
        bool w_ok = true;       // lane l: source rank l / 4, epilogue warp l % 4
        if (lane < p.world * kFlagsPerTile)
          w_ok = wait_ge<true>(my_flags + ((lane / kFlagsPerTile) * p.max_tiles + w) * kFlagsPerTile + (lane % kFlagsPerTile),
                               p.epoch, p.status, 840);
        ok = __all_sync(0xffffffffu, w_ok);
        if (!ok) break;
        const int cols = min(BN, p.N - nb * BN);
        const int vec_per_row = cols / 8;
        for (int v = et; v < BM * vec_per_row; v += 128) {
          const int row = v / vec_per_row, cv = v - row * vec_per_row;
          const long off = ((long)(mb * BM + row)) * row_bytes + ((long)nb * BN + cv * 8) * 2;
          float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int src = 0; src < p.world; ++src) {
            const uint4 u = ld_peer_v4(p.sym[p.rank] + (long)src * p.Tl * row_bytes + off);
            const float2 x0 = unpack_bf16x2(u.x), x1 = unpack_bf16x2(u.y), x2 = unpack_bf16x2(u.z), x3 = unpack_bf16x2(u.w);
            a[0] += x0.x; a[1] += x0.y; a[2] += x1.x; a[3] += x1.y; a[4] += x2.x; a[5] += x2.y; a[6] += x3.x; a[7] += x3.y;
          }
          const int n = nb * BN + cv * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float b = 0.f;
            if (p.bias_kind == 1) b = __ldg((const float*)p.bias + n + j);
            else if (p.bias_kind == 2) b = __bfloat162float(((const __nv_bfloat16*)p.bias)[n + j]);
            a[j] = apply_act(a[j] + b, p.act);
          }
          uint4 o;
          o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
          o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
          *reinterpret_cast<uint4*>(p.out + off) = o;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<C::kTmemCols>(tmem_base);
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
           const CommParams& p, int grid, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_comm_kernel<BN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, kThreads, C::kSmem, stream>>>(ma, mal, mb, mc, p);
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
    mc = ma;
  }
  rc = make_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, (uint32_t)BN);
  if (rc) return 2000 + rc;
  if (BN == 256)
    return mode == MODE_AG ? launch<256, MODE_AG>(ma, mal, mb, mc, p, grid, stream)
                           : launch<256, MODE_RS>(ma, mal, mb, mc, p, grid, stream);
  return mode == MODE_AG ? launch<128, MODE_AG>(ma, mal, mb, mc, p, grid, stream)
                         : launch<128, MODE_RS>(ma, mal, mb, mc, p, grid, stream);
}
