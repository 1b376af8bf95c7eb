// Flash-attention backward for sm_100a (bf16, head_dim 128, causal/full, grouped-query heads).
//
// Two launches of one kernel template share a skeleton (no atomics, deterministic):
//   MODE_DKV: one CTA per (batch, kv head, 128-key block); K,V stay in shared memory, 64-query
//             tiles of Q and dO stream through (all query heads of the group, all visible query
//             blocks).  S^T = K Q^T and dP^T = V dO^T go to TMEM, the compute warps turn them into
//             P^T and dS^T (bf16, shared memory), then dV += P^T dO and dK += dS^T Q accumulate in
//             TMEM.
//   MODE_DQ : one CTA per (batch, query head, 128-query block); Q,dO stay, 64-key tiles of K and V
//             stream; S = Q K^T, dP = dO V^T, dS -> shared memory, dQ += dS K.
// Probabilities are recomputed from the forward's log-sum-exp; delta = rowsum(dO * O) comes from
// a small pre-pass kernel.  Scores are recomputed in both launches (7 GEMM-equivalents instead of
// 5) in exchange for never needing atomic accumulation of dQ.
//
// Warp roles: 0 = TMA, 1 = MMA issue + TMEM owner, 2..17 = compute (each score row is split
// between four threads, 16 of the 64 columns each, so that every SM sub-partition has four compute
// warps to interleave).
//
// The reference has no attention backward at all (its attention builds a fresh leaf,
// crates/axonml-nn/src/layers/attention.rs:225-228); the forward it mirrors is
// crates/axonml-llm/src/attention.rs:836-943.
#include "flash_common.cuh"

namespace {
using namespace ax;
using namespace fa;

constexpr int MODE_DKV = 0, MODE_DQ = 1;
constexpr int BS = 128;                   // rows of the stationary tiles
constexpr int BT = 64;                    // rows of the streamed tiles (= score tile width)
constexpr int kComputeWarps = 16;         // four per TMEM lane quarter: latency of the TMEM loads, exponentials and
                                          // shared-memory stores of one warp hides behind the other three
constexpr int CPT = BT * 4 / kComputeWarps;   // score columns per compute thread
constexpr int kThreads = 64 + kComputeWarps * 32;
constexpr int kStat = BS * HD * 2;        // 32 KB
constexpr int kStream = BT * HD * 2;      // 16 KB
constexpr int kETile = BS * BT * 2;       // 16 KB
constexpr int kStages = 3;                // streamed-tile stages: a stage is released by the accumulate MMAs of
                                          // its tile, so two stages put the TMA latency of tile t+1 in series
                                          // with the accumulate of tile t-1 (660 -> 554 us at B4 H16 S2048)
constexpr int kLseBytes = kComputeWarps * 2 * CPT * 4; // per compute warp: the scaled log-sum-exps and deltas of its columns
constexpr int kSmem = 1024 + 2 * kStat + kStages * 2 * kStream + 2 * kETile + kLseBytes + 256;
constexpr int kTmemCols = 512;            // T1[0] T2[0] T1[1] T2[1] (64 each) | acc1 (128) | acc2 (128)
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  const float* lse;     // [B, Hq, Sq]
  const float* delta;   // [B, Hq, Sq]
  void* out1;           // DKV: dV [B,Skv,Hkv,D];  DQ: unused
  void* out2;           // DKV: dK [B,Skv,Hkv,D];  DQ: dQ [B,Sq,Hq,D]
  long o_row, o_batch;  // strides (elements) of out1/out2
  int B, Hq, Hkv, Sq, Skv, causal;
  float scale, scale_log2;
  int* status;
};

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap map_a1, const __grid_constant__ CUtensorMap map_a2,
                 const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_b2,
                 const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA1 = smem;
  uint8_t* sA2 = sA1 + kStat;
  uint8_t* sB = sA2 + kStat;               // stage s: B1 at sB + s*2*kStream, B2 right after it
  uint8_t* sE1 = sB + kStages * 2 * kStream;
  uint8_t* sE2 = sE1 + kETile;
  float* sLse = (float*)(sE2 + kETile);   // [compute warp][log-sum-exps | deltas][CPT]
  uint64_t* bars = (uint64_t*)((uint8_t*)sLse + kLseBytes);
  uint64_t* stat_full = bars;        // 1
  uint64_t* b_full = bars + 1;       // kStages
  uint64_t* b_empty = bars + 4;      // kStages
  uint64_t* t_full = bars + 7;       // 2
  uint64_t* t_empty = bars + 9;      // 2
  uint64_t* e_full = bars + 11;      // 1
  uint64_t* e_free = bars + 12;      // 1
  uint32_t* tmem_slot = (uint32_t*)(bars + 13);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One-dimensional grid, longest CTAs first: with a causal mask a key block early in the sequence (DKV) or a
  // query block late in it (DQ) sees the most tiles, and CTAs are handed out in index order, so the block index
  // is the slow coordinate and (head, batch) the fast one.
  const int nblk = (int)gridDim.x / (p.B * ((MODE == MODE_DQ) ? p.Hq : p.Hkv));
  const int slow = (int)blockIdx.x / (p.B * ((MODE == MODE_DQ) ? p.Hq : p.Hkv));
  const int fast = (int)blockIdx.x - slow * (p.B * ((MODE == MODE_DQ) ? p.Hq : p.Hkv));
  const int blk = (MODE == MODE_DQ) ? (nblk - 1 - slow) : slow;
  const int hh = fast % ((MODE == MODE_DQ) ? p.Hq : p.Hkv);   // DKV: hh = kv head; DQ: hh = query head
  const int b = fast / ((MODE == MODE_DQ) ? p.Hq : p.Hkv);
  const int G = p.Hq / p.Hkv;
  const int offset = p.Skv - p.Sq;
  const int row0 = blk * BS;                       // first stationary row (key or query index)

  // iteration space of streamed tiles
  int T, first_tile = 0, tiles_per_head = 0;
  if (MODE == MODE_DKV) {
    const int nq = (p.Sq + BT - 1) / BT;
    if (p.causal) {
      int qmin = row0 - offset;                    // first query that can see key row0
      first_tile = qmin > 0 ? qmin / BT : 0;
    }
    tiles_per_head = nq - first_tile;
    if (tiles_per_head < 0) tiles_per_head = 0;
    T = tiles_per_head * G;
  } else {
    int kv_end = p.Skv;
    if (p.causal) kv_end = min(p.Skv, row0 + BS + offset);
    T = kv_end > 0 ? (kv_end + BT - 1) / BT : 0;
  }

  if (threadIdx.x == 0) {
    *dead = 0;
    mbar_init(stat_full, 1);
    for (int i = 0; i < kStages; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], kComputeWarps); }
    mbar_init(e_full, kComputeWarps);
    mbar_init(e_free, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<kTmemCols>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tAcc1 = tmem_base + 256, tAcc2 = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0 && T > 0) {
      const int hs = (MODE == MODE_DKV) ? hh : hh;                 // head of the stationary tiles
      mbar_expect_tx(stat_full, 2 * kStat);
      tma_load_4d(sA1, &map_a1, stat_full, 0, hs, row0, b);
      tma_load_4d(sA1 + slab_bytes(BS), &map_a1, stat_full, 64, hs, row0, b);
      tma_load_4d(sA2, &map_a2, stat_full, 0, hs, row0, b);
      tma_load_4d(sA2 + slab_bytes(BS), &map_a2, stat_full, 64, hs, row0, b);
      for (int t = 0; t < T; ++t) {
        const int s = t % kStages;
        const uint32_t ph = (t / kStages) & 1;
        int head, r0;
        if (MODE == MODE_DKV) {
          const int g = t / tiles_per_head;
          head = hh * G + g;
          r0 = (first_tile + (t - g * tiles_per_head)) * BT;
        } else {
          head = hh / G;
          r0 = t * BT;
        }
        if (!mbar_wait(&b_empty[s], ph ^ 1, dead, p.status, 500)) break;
        uint8_t* d1 = sB + s * 2 * kStream;
        uint8_t* d2 = d1 + kStream;
        mbar_expect_tx(&b_full[s], 2 * kStream);
        tma_load_4d(d1, &map_b1, &b_full[s], 0, head, r0, b);
        tma_load_4d(d1 + slab_bytes(BT), &map_b1, &b_full[s], 64, head, r0, b);
        tma_load_4d(d2, &map_b2, &b_full[s], 0, head, r0, b);
        tma_load_4d(d2 + slab_bytes(BT), &map_b2, &b_full[s], 64, head, r0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && T > 0) {
      constexpr uint32_t idesc_t = umma_idesc_f16(1, 128, 64, 0, 0);
      constexpr uint32_t idesc_a = umma_idesc_f16(1, 128, 128, 0, 1);
      const uint32_t aA1 = smem_u32(sA1), aA2 = smem_u32(sA2);
      const uint32_t aE1 = smem_u32(sE1), aE2 = smem_u32(sE2);
      bool ok = mbar_wait(stat_full, 0, dead, p.status, 510);
      auto issue_scores = [&](int t) {
        const int s = t & 1, bs = t % kStages;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&b_full[bs], (t / kStages) & 1, dead, p.status, 511)) return false;
        if (!mbar_wait(&t_empty[s], ph ^ 1, dead, p.status, 512)) return false;
        tc_fence_after();
        const uint32_t aB1 = smem_u32(sB + bs * 2 * kStream), aB2 = aB1 + kStream;
        const uint32_t tT1 = tmem_base + s * 128, tT2 = tT1 + 64;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ss(tT1, desc_kmajor(aA1, BS, k), desc_kmajor(aB1, BT, k), idesc_t, k != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ss(tT2, desc_kmajor(aA2, BS, k), desc_kmajor(aB2, BT, k), idesc_t, k != 0);
        umma_commit(&t_full[s]);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int t = 0; ok && t < T; ++t) {
        if (t + 1 < T) ok = issue_scores(t + 1);
        if (!ok) break;
        const int s = t % kStages;
        if (!mbar_wait(e_full, t & 1, dead, p.status, 513)) break;
        tc_fence_after();
        const uint32_t aB1 = smem_u32(sB + s * 2 * kStream), aB2 = aB1 + kStream;
        if (MODE == MODE_DKV) {
#pragma unroll
          for (int k = 0; k < 4; ++k)   // dV += P^T dO
            umma_f16_ss(tAcc1, umma_desc_sw128(aE1 + k * 32, 16, 1024), desc_mnmajor(aB2, BT, k), idesc_a, (t | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)     // DKV: dK += dS^T Q;  DQ: dQ += dS K
          umma_f16_ss(tAcc2, umma_desc_sw128(aE2 + k * 32, 16, 1024), desc_mnmajor(aB1, BT, k), idesc_a, (t | k) != 0);
        umma_commit(&b_empty[s]);
        umma_commit(e_free);
      }
    }
  } else {
    const int cw = warp - 2;
    const int q = warp & 3;                         // TMEM lane quarter
    const int part = cw >> 2;                       // which CPT of the 64 score columns
    const int r = q * 32 + lane;                    // stationary row inside the tile
    const int ri = row0 + r;                        // its key (DKV) or query (DQ) index
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float lse_r = 0.f, delta_r = 0.f;
    if (MODE == MODE_DQ) {
      const bool v = ri < p.Sq;
      const long idx = ((long)b * p.Hq + hh) * p.Sq + ri;
      lse_r = v ? p.lse[idx] * kLog2e : INFINITY;
      delta_r = v ? p.delta[idx] : 0.f;
    }
    // DKV: the columns of a score tile are queries, so every lane of a warp needs the same CPT
    // log-sum-exps and deltas.  Lanes 0..15 fetch the scaled log-sum-exps of the warp's columns one
    // tile ahead, lanes 16..31 the deltas (one coalesced load), the warp parks them in its own slice
    // of shared memory and reads them back as broadcast float4s.  A column past Sq gets an infinite
    // log-sum-exp, i.e. probability zero.
    float* my_lse = sLse + cw * 32;
    float nstat = 0.f;
    auto fetch_cols = [&](int t) {
      const int g = t / tiles_per_head;
      const int qi = (first_tile + (t - g * tiles_per_head)) * BT + part * CPT + (lane & (CPT - 1));
      const long idx = ((long)b * p.Hq + hh * G + g) * p.Sq + qi;
      const bool v = qi < p.Sq;
      if (lane < CPT) nstat = v ? __ldg(p.lse + idx) * kLog2e : INFINITY;
      else nstat = v ? __ldg(p.delta + idx) : 0.f;
    };
    if (MODE == MODE_DKV && T > 0) fetch_cols(0);
    bool ok = true;
    for (int t = 0; t < T && ok; ++t) {
      const int s = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      int c0;
      bool need_mask;                               // warp-uniform: some (row, column) of this warp is hidden
      if (MODE == MODE_DKV) {
        const int g = t / tiles_per_head;
        c0 = (first_tile + (t - g * tiles_per_head)) * BT + part * CPT;   // first query of my columns
        need_mask = p.causal && c0 < row0 + q * 32 + 31 - offset;
        __syncwarp();                                                    // the previous tile's reads are done
        my_lse[lane] = nstat;
        if (t + 1 < T) fetch_cols(t + 1);
        __syncwarp();
      } else {
        c0 = t * BT + part * CPT;                                        // first key of my columns
        const int min_limit = p.causal ? min(p.Skv - 1, row0 + q * 32 + offset) : p.Skv - 1;
        need_mask = c0 + CPT - 1 > min_limit;
      }
      ok = mbar_wait(&t_full[s], ph, dead, p.status, 520);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[CPT], dv[CPT];
      tmem_ld_32x32b_x16(tmem_base + s * 128 + part * CPT + lane_addr, sv);
      tmem_ld_32x32b_x16(tmem_base + s * 128 + 64 + part * CPT + lane_addr, dv);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&t_empty[s]);

      float pr[CPT], ds[CPT];
      if (MODE == MODE_DQ) {
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          pr[i] = exp2f(__uint_as_float(sv[i]) * p.scale_log2 - lse_r);
          ds[i] = pr[i] * (__uint_as_float(dv[i]) - delta_r);
        }
        if (need_mask) {
          const int limit = p.causal ? min(p.Skv - 1, ri + offset) : p.Skv - 1;
#pragma unroll
          for (int i = 0; i < CPT; ++i)
            if (c0 + i > limit) { pr[i] = 0.f; ds[i] = 0.f; }
        }
      } else {
#pragma unroll
        for (int i4 = 0; i4 < CPT / 4; ++i4) {
          const float4 l4 = *reinterpret_cast<const float4*>(my_lse + i4 * 4);
          const float4 d4 = *reinterpret_cast<const float4*>(my_lse + CPT + i4 * 4);
          const float l[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = i4 * 4 + j;
            pr[i] = exp2f(__uint_as_float(sv[i]) * p.scale_log2 - l[j]);
            ds[i] = pr[i] * (__uint_as_float(dv[i]) - dl[j]);
          }
        }
        if (need_mask) {
          const int first_visible = ri - offset;    // the causal rule hides queries before key ri - offset
#pragma unroll
          for (int i = 0; i < CPT; ++i)
            if (c0 + i < first_visible) { pr[i] = 0.f; ds[i] = 0.f; }
        }
      }
      // the E tiles are free once the accumulate MMAs of the previous tile have retired
      if (t > 0) {
        ok = mbar_wait(e_free, (t - 1) & 1, dead, p.status, 521);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int g4 = 0; g4 < CPT / 8; ++g4) {
        uint4 o;
        if (MODE == MODE_DKV) {
          o.x = pack_bf16x2(pr[g4 * 8 + 0], pr[g4 * 8 + 1]); o.y = pack_bf16x2(pr[g4 * 8 + 2], pr[g4 * 8 + 3]);
          o.z = pack_bf16x2(pr[g4 * 8 + 4], pr[g4 * 8 + 5]); o.w = pack_bf16x2(pr[g4 * 8 + 6], pr[g4 * 8 + 7]);
          store_tile_chunk(sE1, BS, r, part * (CPT / 8) + g4, o);
        }
        o.x = pack_bf16x2(ds[g4 * 8 + 0], ds[g4 * 8 + 1]); o.y = pack_bf16x2(ds[g4 * 8 + 2], ds[g4 * 8 + 3]);
        o.z = pack_bf16x2(ds[g4 * 8 + 4], ds[g4 * 8 + 5]); o.w = pack_bf16x2(ds[g4 * 8 + 6], ds[g4 * 8 + 7]);
        store_tile_chunk(sE2, BS, r, part * (CPT / 8) + g4, o);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(e_full);
    }
    // epilogue: accumulators -> global (this thread: row ri, columns [part*32, part*32+32))
    if (ok && T > 0) {
      ok = mbar_wait(e_free, (T - 1) & 1, dead, p.status, 522);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const int rows_total = (MODE == MODE_DKV) ? p.Skv : p.Sq;
      const bool valid = ri < rows_total;
      constexpr int kCols = HD / (kComputeWarps / 4);            // 32 output columns per thread
      static_assert(kCols == 32, "the epilogue reads one 32-column TMEM chunk per accumulator");
      const long base = (long)b * p.o_batch + (long)ri * p.o_row + (long)hh * HD + part * kCols;
#pragma unroll 1
      for (int which = (MODE == MODE_DKV ? 0 : 1); which < 2; ++which) {
        __nv_bfloat16* orow = (__nv_bfloat16*)(which == 0 ? p.out1 : p.out2) + base;
        const uint32_t tacc = (which == 0 ? tAcc1 : tAcc2) + lane_addr + part * kCols;
        const float mul = which == 0 ? 1.f : p.scale;
        uint32_t v[32];
        if (T > 0) {
          tmem_ld_32x32b_x32(tacc, v);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (valid) {
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[g4 * 8 + 0]) * mul, __uint_as_float(v[g4 * 8 + 1]) * mul);
            o.y = pack_bf16x2(__uint_as_float(v[g4 * 8 + 2]) * mul, __uint_as_float(v[g4 * 8 + 3]) * mul);
            o.z = pack_bf16x2(__uint_as_float(v[g4 * 8 + 4]) * mul, __uint_as_float(v[g4 * 8 + 5]) * mul);
            o.w = pack_bf16x2(__uint_as_float(v[g4 * 8 + 6]) * mul, __uint_as_float(v[g4 * 8 + 7]) * mul);
            *reinterpret_cast<uint4*>(orow + g4 * 8) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<kTmemCols>(tmem_base);
}

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d]; one warp per (b,s,h)
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                   float* __restrict__ delta, int B, int S, int H, long o_row, long o_batch,
                                   long do_row, long do_batch) {
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = (long)B * S * H;
  if (w >= total) return;
  const int h = (int)(w % H);
  const long bs = w / H;
  const int s = (int)(bs % S);
  const int b = (int)(bs / S);
  const uint2 a = *reinterpret_cast<const uint2*>(o + b * o_batch + s * o_row + (long)h * HD + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(dout + b * do_batch + s * do_row + (long)h * HD + lane * 4);
  float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y);
  float acc = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
  acc = warp_sum(acc);
  if (lane == 0) delta[((long)b * H + h) * S + s] = acc;
}

template <int MODE>
int launch_bwd(dim3 grid, const CUtensorMap& a1, const CUtensorMap& a2, const CUtensorMap& b1, const CUtensorMap& b2,
               const BwdParams& p, cudaStream_t stream) {
  auto kern = flash_bwd_kernel<MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, kThreads, kSmem, stream>>>(a1, a2, b1, b2, p);
  return (int)cudaGetLastError();
}

}  // namespace

// All tensors token-major [B, S, H, 128] bf16; strides in elements.  dq/dk/dv are written densely
// with the given output strides.  delta is scratch [B, Hq, Sq] fp32 provided by the caller.
AX_API int ax_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                        const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int Sq,
                        int Skv, int Hq, int Hkv, int D, long q_row, long q_batch, long k_row,
                        long k_batch, long v_row, long v_batch, long o_row, long o_batch, long do_row,
                        long do_batch, long dq_row, long dq_batch, long dkv_row, long dkv_batch,
                        int causal, float scale, int* status, cudaStream_t stream) {
  if (D != fa::HD || Hq % Hkv != 0) return -1;
  if ((q_row | k_row | v_row | o_row | do_row | dq_row | dkv_row) % 8) return -1;
  if (B <= 0 || Sq <= 0 || Skv <= 0) return 0;
  {
    long warps = (long)B * Sq * Hq;
    int block = 256;
    long grid = (warps * 32 + block - 1) / block;
    flash_delta_kernel<<<(unsigned)grid, block, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                             delta, B, Sq, Hq, o_row, o_batch, do_row, do_batch);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  CUtensorMap mq128, mdo128, mk128, mv128, mq64, mdo64, mk64, mv64;
  int rc;
  if ((rc = axh::make_bshd_map(&mq128, q, D, Hq, Sq, B, q_row, q_batch, BS))) return 1000 + rc;
  if ((rc = axh::make_bshd_map(&mdo128, dout, D, Hq, Sq, B, do_row, do_batch, BS))) return 1100 + rc;
  if ((rc = axh::make_bshd_map(&mk128, k, D, Hkv, Skv, B, k_row, k_batch, BS))) return 1200 + rc;
  if ((rc = axh::make_bshd_map(&mv128, v, D, Hkv, Skv, B, v_row, v_batch, BS))) return 1300 + rc;
  if ((rc = axh::make_bshd_map(&mq64, q, D, Hq, Sq, B, q_row, q_batch, BT))) return 1400 + rc;
  if ((rc = axh::make_bshd_map(&mdo64, dout, D, Hq, Sq, B, do_row, do_batch, BT))) return 1500 + rc;
  if ((rc = axh::make_bshd_map(&mk64, k, D, Hkv, Skv, B, k_row, k_batch, BT))) return 1600 + rc;
  if ((rc = axh::make_bshd_map(&mv64, v, D, Hkv, Skv, B, v_row, v_batch, BT))) return 1700 + rc;

  BwdParams p;
  p.lse = lse; p.delta = delta;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.status = status;
  // dK, dV
  p.out1 = dv; p.out2 = dk; p.o_row = dkv_row; p.o_batch = dkv_batch;
  dim3 g1(((Skv + BS - 1) / BS) * Hkv * B, 1, 1);
  int e = launch_bwd<MODE_DKV>(g1, mk128, mv128, mq64, mdo64, p, stream);
  if (e != 0) return e;
  // dQ
  p.out1 = nullptr; p.out2 = dq; p.o_row = dq_row; p.o_batch = dq_batch;
  dim3 g2(((Sq + BS - 1) / BS) * Hq * B, 1, 1);
  return launch_bwd<MODE_DQ>(g2, mq128, mdo128, mk64, mv64, p, stream);
}
