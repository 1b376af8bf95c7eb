// Flash-attention forward for sm_100a: bf16, head_dim 128, causal or full, grouped-query heads,
// token-major [B, S, H, D] operands (views into a fused QKV tensor are fine).
//
// One CTA per (batch, query head, 128-query block).  Warp 0 streams K/V blocks of 128 keys with
// TMA (two stages), warp 1 issues tcgen05.mma: S = Q K^T into one of two TMEM buffers and
// O += P V into a TMEM accumulator, warps 2..5 (one thread per query row) read S from TMEM, keep
// the running max / sum, write P as bf16 into one of two shared-memory buffers for the second MMA
// (so softmax(j+1) does not wait for P(j) V(j)), and rescale O in
// TMEM only when a row's max has grown by more than 2^8 (the deferred-rescale trick keeps the
// result exact because the final normalisation uses the same reference max).  S(j+1) is issued
// before P(j) V(j), so the tensor pipe works on the next block while softmax(j) runs.
//
// Parity: FlashAttention forward crates/axonml-llm/src/attention.rs:836-943 (CPU, block 64) and
// the attention inside LLaMA / GPT-2 (llama.rs:429-441).
#include "flash_common.cuh"

namespace {
using namespace ax;
using namespace fa;

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kThreads = 192;
constexpr int kTile = BQ * HD * 2;           // 32 KB: one [128 x 128] bf16 tile
constexpr int kSmem = 1024 + kTile /*Q*/ + 2 * kTile /*K*/ + 2 * kTile /*V*/ + 2 * kTile /*P*/ + 256;
constexpr int kTmemCols = 512;               // S0 | S1 | O | (unused)
constexpr float kRescaleThreshold = 8.0f;    // log2 units

struct FwdParams {
  void* out;          // [B, Sq, Hq, D] bf16
  long o_row_stride, o_batch_stride;
  float* lse;         // [B, Hq, Sq] natural-log log-sum-exp
  int B, Hq, Hkv, Sq, Skv;
  int causal;
  float scale_log2;   // softmax scale * log2(e)
  int* status;
  unsigned long long* trace;   // optional timeline of two CTAs ([2][kTraceSlots] globaltimer stamps), or null
};

// Timeline: slot 0 kernel start, then per KV block five stamps (scores ready, scores in registers,
// max / rescale done, P buffer free, P published), last slot epilogue done.
constexpr int kTraceSlots = 128;

__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTile;
  uint8_t* sV = sK + 2 * kTile;
  uint8_t* sP = sV + 2 * kTile;
  uint64_t* bars = (uint64_t*)(sP + 2 * kTile);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* s_empty = bars + 11;    // 2
  uint64_t* p_full = bars + 13;     // 2 (one per P buffer)
  uint64_t* pv_done = bars + 15;    // 2 (P V of even / odd blocks)
  uint32_t* tmem_slot = (uint32_t*)(bars + 17);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one-dimensional grid, handed out in index order: the query block is the slow coordinate, so the
  // longest (last) query blocks of every head start first and the short ones fill the tail
  const int slow = (int)blockIdx.x / (p.Hq * p.B), fast = (int)blockIdx.x - slow * (p.Hq * p.B);
  const int qb = (int)gridDim.x / (p.Hq * p.B) - 1 - slow;
  const int h = fast % p.Hq, b = fast / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * BQ;
  const int offset = p.Skv - p.Sq;                        // causal: row i sees keys <= i + offset
  int kv_end = p.Skv;
  if (p.causal) kv_end = min(p.Skv, q0 + BQ + offset);
  const int nblk = kv_end > 0 ? (kv_end + BKV - 1) / BKV : 0;

  if (threadIdx.x == 0) {
    *dead = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&p_full[i], 4); mbar_init(&pv_done[i], 1); }
    mbar_fence_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v);
  }
  if (warp == 1) { tmem_alloc<kTmemCols>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base, tO = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      mbar_expect_tx(q_full, kTile);
      tma_load_4d(sQ, &map_q, q_full, 0, h, q0, b);
      tma_load_4d(sQ + slab_bytes(BQ), &map_q, q_full, 64, h, q0, b);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kv0 = j * BKV;
        if (!mbar_wait(&k_empty[s], ph ^ 1, dead, p.status, 400)) break;
        mbar_expect_tx(&k_full[s], kTile);
        tma_load_4d(sK + s * kTile, &map_k, &k_full[s], 0, hk, kv0, b);
        tma_load_4d(sK + s * kTile + slab_bytes(BKV), &map_k, &k_full[s], 64, hk, kv0, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, dead, p.status, 401)) break;
        mbar_expect_tx(&v_full[s], kTile);
        tma_load_4d(sV + s * kTile, &map_v, &v_full[s], 0, hk, kv0, b);
        tma_load_4d(sV + s * kTile + slab_bytes(BKV), &map_v, &v_full[s], 64, hk, kv0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(1, 128, 128, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_f16(1, 128, 128, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, dead, p.status, 410);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph, dead, p.status, 411)) return false;
        if (!mbar_wait(&s_empty[s], ph ^ 1, dead, p.status, 412)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + s * kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ss(tS0 + s * 128, desc_kmajor(aQ, BQ, k), desc_kmajor(aK, BKV, k), idesc_s, k != 0);
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < nblk; ++j) {
        if (j + 1 < nblk) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&p_full[s], ph, dead, p.status, 413)) break;
        if (!mbar_wait(&v_full[s], ph, dead, p.status, 414)) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + s * kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ss(tO, desc_kmajor(aP + s * kTile, BQ, k), desc_mnmajor(aV, BKV, k), idesc_o, (j | k) != 0);
        umma_commit(&v_empty[s]);
        umma_commit(&pv_done[s]);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // row inside the tile == TMEM lane
    const int qi = q0 + r;                       // query index
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t sP_u32 = smem_u32(sP);
    unsigned long long* tr = nullptr;
    if (p.trace != nullptr && warp == 2 && lane == 0 && slow == 0 &&
        ((h == 0 && b == 0) || (h == p.Hq - 1 && b == p.B - 1)))
      tr = p.trace + (b == 0 && h == 0 ? 0 : kTraceSlots);
    auto stamp = [&](int slot) { if (tr != nullptr && slot < kTraceSlots) tr[slot] = globaltimer_ns(); };
    stamp(0);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int kv0 = j * BKV;
      ok = mbar_wait(&s_full[s], ph, dead, p.status, 420);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      stamp(1 + 5 * j);
      // the row's 128 scores, read once: four loads in flight, one wait
      uint32_t v[128];
      {
        const uint32_t tS = tS0 + s * 128 + lane_addr;
        tmem_ld_32x32b_x32(tS, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tmem_ld_32x32b_x32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        tmem_ld_32x32b_x32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&v[64]));
        tmem_ld_32x32b_x32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&v[96]));
        tc_wait_ld();
      }
      // S[s] lives in registers now: hand the TMEM buffer back so that S(j+2) can be issued
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
      stamp(2 + 5 * j);
      const int limit = p.causal ? min(p.Skv - 1, qi + offset) : p.Skv - 1;   // last visible key
      if (__any_sync(0xffffffffu, kv0 + BKV - 1 > limit)) {
        // only blocks that touch the diagonal or the end of the keys pay for the comparison;
        // a masked score becomes -inf, whose probability below is exactly 0
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (kv0 + i > limit) v[i] = 0xff800000u;
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
      float m_new = fmaxf(m, mx * p.scale_log2);
      if (m_new == -INFINITY) m_new = 0.f;
      const bool grow = m_new > m + kRescaleThreshold;
      if (j == 0) {
        m = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        // O may only be touched once every P V issued so far has retired
        ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, dead, p.status, 421);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const float alpha = grow ? exp2f(m - m_new) : 1.f;
        if (grow) { l *= alpha; m = m_new; }
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tO + lane_addr + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x16(tO + lane_addr + c * 16, o);
        }
        tc_wait_st();
        tc_fence_before();
      }
      if (tr != nullptr) { asm volatile("" ::"f"(m), "f"(mx) : "memory"); }
      stamp(3 + 5 * j);
      // P buffer s was last read by P V of block j-2
      if (j >= 2) {
        ok = mbar_wait(&pv_done[s], ((j - 2) >> 1) & 1, dead, p.status, 423);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      stamp(4 + 5 * j);
      // probabilities -> shared memory (bf16, the swizzled K-major operand of P V), row sum
      const uint32_t sp_row = sP_u32 + s * kTile + r * 128;
      const float neg_m = -m;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2f(fmaf(__uint_as_float(v[c * 8 + i]), p.scale_log2, neg_m));
          rs += e[i];
        }
        const uint32_t addr = sp_row + (c >> 3) * slab_bytes(BQ) + (((c & 7) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_bf16x2(e[0], e[1])),
                     "r"(pack_bf16x2(e[2], e[3])), "r"(pack_bf16x2(e[4], e[5])), "r"(pack_bf16x2(e[6], e[7]))
                     : "memory");
      }
      l += rs;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
      stamp(5 + 5 * j);
    }
    // epilogue: O / l -> global, lse
    if (ok && nblk > 0) {
      ok = mbar_wait(&pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, dead, p.status, 422);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool valid = qi < p.Sq;
      __nv_bfloat16* orow = (__nv_bfloat16*)p.out + (long)b * p.o_batch_stride + (long)qi * p.o_row_stride + (long)h * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (nblk > 0) {
          tmem_ld_32x32b_x32(tO + lane_addr + c * 32, v);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
          }
        }
      }
      if (valid && p.lse)
        p.lse[((long)b * p.Hq + h) * p.Sq + qi] = l > 0.f ? (m * 0.6931471805599453f + logf(l)) : -INFINITY;
      stamp(kTraceSlots - 1);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<kTmemCols>(tmem_base);
}


// ------------------------------------------------------------------------------------------
// Two query tiles per CTA.  The exponentials of a 128 x 128 score block take the SM's special-
// function units about as long as its two MMAs take the tensor pipe, so one tile alone leaves
// each unit idle half of the time.  Here a CTA owns 256 query rows as tiles A and B with a softmax
// warpgroup each: while one tile's probabilities are computed the tensor pipe works on the other
// tile.  Probabilities never touch shared memory: they are written back as packed bf16 into the
// first 64 TMEM columns of the tile's score buffer and the second MMA takes them from there (A
// operand in TMEM), which also frees shared memory for the two Q tiles.
//   TMEM: S_A | S_B | O_A | O_B, 128 columns each.
//   warp 0: TMA (Q once, K/V blocks through two stages); warp 1: MMA; warps 2..5: softmax of tile
//   A; warps 6..9: softmax of tile B (a warp may touch TMEM lanes 32 (w % 4) .. +31 only, which is
//   why both groups start at a multiple of four plus two).
constexpr int kThreads2 = 320;
constexpr int kSmem2 = 1024 + 2 * kTile /*Q A,B*/ + 2 * kTile /*K*/ + 2 * kTile /*V*/ + 256;

template <bool kTrace>
__global__ void __launch_bounds__(kThreads2, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                 // [2][128 x 128]
  uint8_t* sK = sQ + 2 * kTile;       // [2 stages]
  uint8_t* sV = sK + 2 * kTile;
  uint64_t* bars = (uint64_t*)(sV + 2 * kTile);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // [tile]: scores of the tile's next block are in TMEM
  uint64_t* p_full = bars + 11;       // [tile]: its probabilities are in TMEM (4 warps arrive)
  uint64_t* pv_done = bars + 13;      // [tile]: every P V issued so far for the tile has retired
  uint32_t* tmem_slot = (uint32_t*)(bars + 15);
  volatile int* dead = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one-dimensional grid with the query block as the slow coordinate: longest CTAs first
  const int slow = (int)blockIdx.x / (p.Hq * p.B), fast = (int)blockIdx.x - slow * (p.Hq * p.B);
  const int qb = (int)gridDim.x / (p.Hq * p.B) - 1 - slow;
  const int h = fast % p.Hq, b = fast / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * 2 * BQ;
  const int offset = p.Skv - p.Sq;                        // causal: row i sees keys <= i + offset
  int nblk_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    int kv_end = p.Skv;
    if (p.causal) kv_end = min(p.Skv, q0 + (t + 1) * BQ + offset);
    if (q0 + t * BQ >= p.Sq) kv_end = 0;                  // no query row of this tile exists
    nblk_t[t] = kv_end > 0 ? (kv_end + BKV - 1) / BKV : 0;
  }
  const int nblk = max(nblk_t[0], nblk_t[1]);

  if (threadIdx.x == 0) {
    *dead = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&pv_done[i], 1);
    }
    mbar_fence_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v);
  }
  if (warp == 1) { tmem_alloc<kTmemCols>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      mbar_expect_tx(q_full, 2 * kTile);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        tma_load_4d(sQ + t * kTile, &map_q, q_full, 0, h, q0 + t * BQ, b);
        tma_load_4d(sQ + t * kTile + slab_bytes(BQ), &map_q, q_full, 64, h, q0 + t * BQ, b);
      }
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kv0 = j * BKV;
        if (!mbar_wait(&k_empty[s], ph ^ 1, dead, p.status, 430)) break;
        mbar_expect_tx(&k_full[s], kTile);
        tma_load_4d(sK + s * kTile, &map_k, &k_full[s], 0, hk, kv0, b);
        tma_load_4d(sK + s * kTile + slab_bytes(BKV), &map_k, &k_full[s], 64, hk, kv0, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, dead, p.status, 431)) break;
        mbar_expect_tx(&v_full[s], kTile);
        tma_load_4d(sV + s * kTile, &map_v, &v_full[s], 0, hk, kv0, b);
        tma_load_4d(sV + s * kTile + slab_bytes(BKV), &map_v, &v_full[s], 64, hk, kv0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(1, 128, 128, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_f16(1, 128, 128, 0, 1);
      const uint32_t aQ = smem_u32(sQ);
      bool ok = mbar_wait(q_full, 0, dead, p.status, 440);
      // S_t(j) = Q_t K_j^T into the tile's score columns
      auto issue_s = [&](int t, int j) {
        const uint32_t aK = smem_u32(sK + (j & 1) * kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ss(tmem_base + t * 128, desc_kmajor(aQ + t * kTile, BQ, k), desc_kmajor(aK, BKV, k), idesc_s, k != 0);
        umma_commit(&s_full[t]);
      };
      // both tiles' scores of block j (K_j must have landed); K's stage is free afterwards
      auto issue_s_both = [&](int j) {
        if (!mbar_wait(&k_full[j & 1], (j >> 1) & 1, dead, p.status, 441)) return false;
        tc_fence_after();
        if (j < nblk_t[0]) issue_s(0, j);
        if (j < nblk_t[1]) issue_s(1, j);
        umma_commit(&k_empty[j & 1]);
        return true;
      };
      if (ok) ok = issue_s_both(0);
      for (int j = 0; ok && j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&v_full[s], (j >> 1) & 1, dead, p.status, 442)) break;
        const uint32_t aV = smem_u32(sV + s * kTile);
        const bool more = j + 1 < nblk;
        if (more && !mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, dead, p.status, 443)) break;
        const uint32_t aK1 = smem_u32(sK + ((j + 1) & 1) * kTile);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= nblk_t[t]) continue;
          // O_t += P_t(j) V_j with P read from TMEM, then at once the tile's next scores: they
          // overwrite the columns P occupies, which the in-order tensor pipe reads first
          if (!mbar_wait(&p_full[t], j & 1, dead, p.status, 444)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8, desc_mnmajor(aV, BKV, k), idesc_o, (j | k) != 0);
          umma_commit(&pv_done[t]);
          if (j + 1 < nblk_t[t]) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_f16_ss(tmem_base + t * 128, desc_kmajor(aQ + t * kTile, BQ, k), desc_kmajor(aK1, BKV, k), idesc_s, k != 0);
            umma_commit(&s_full[t]);
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[s]);
        if (more) umma_commit(&k_empty[(j + 1) & 1]);
      }
    }
  } else {
    const int t = (warp - 2) >> 2;               // tile of this warpgroup
    const int q = warp & 3;                      // TMEM lane quarter
    const int r = q * 32 + lane;                 // row inside the tile == TMEM lane
    const int qi = q0 + t * BQ + r;              // query index
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_addr;
    const uint32_t tO = tmem_base + 256 + t * 128 + lane_addr;
    const int my_blk = nblk_t[t];
    // timeline of the first CTA (the longest one of head 0, batch 0): quarter-0 warp of tile A in
    // slot row 0, of tile B in row 1; five stamps per KV block
    unsigned long long* tr = nullptr;
    if (kTrace && p.trace != nullptr && q == 0 && lane == 0 && blockIdx.x == 0) tr = p.trace + t * kTraceSlots;
    auto stamp = [&](int slot) { if (kTrace && tr != nullptr && slot < kTraceSlots) tr[slot] = globaltimer_ns(); };
    stamp(0);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_blk && ok; ++j) {
      const int kv0 = j * BKV;
      ok = mbar_wait(&s_full[t], j & 1, dead, p.status, 450);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      stamp(1 + 5 * j);
      uint32_t v[128];
      tmem_ld_32x32b_x32(tS, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld_32x32b_x32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_ld_32x32b_x32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&v[64]));
      tmem_ld_32x32b_x32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&v[96]));
      tc_wait_ld();
      stamp(2 + 5 * j);
      const int limit = p.causal ? min(p.Skv - 1, qi + offset) : p.Skv - 1;   // last visible key
      if (__any_sync(0xffffffffu, kv0 + BKV - 1 > limit)) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (kv0 + i > limit) v[i] = 0xff800000u;
      }
      // four independent chains each (a single running max or sum is a 128-deep dependency chain
      // that the other tile's warp on this scheduler cannot hide)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx4[0] = fmaxf(mx4[0], __uint_as_float(v[i]));
        mx4[1] = fmaxf(mx4[1], __uint_as_float(v[i + 1]));
        mx4[2] = fmaxf(mx4[2], __uint_as_float(v[i + 2]));
        mx4[3] = fmaxf(mx4[3], __uint_as_float(v[i + 3]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float m_new = fmaxf(m, mx * p.scale_log2);
      if (m_new == -INFINITY) m_new = 0.f;
      const bool grow = m_new > m + kRescaleThreshold;
      if (j == 0) {
        m = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        // O may only be touched once every P V issued so far for this tile has retired
        ok = mbar_wait(&pv_done[t], (j - 1) & 1, dead, p.status, 451);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const float alpha = grow ? exp2f(m - m_new) : 1.f;
        if (grow) { l *= alpha; m = m_new; }
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tO + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x16(tO + c * 16, o);
        }
        tc_wait_st();
      }
      stamp(3 + 5 * j);
      // probabilities as packed bf16 pairs into the first 64 score columns, row sum in fp32
      const float neg_m = -m;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float e0 = exp2f(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, neg_m));
        const float e1 = exp2f(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, neg_m));
        rs4[i & 3] += e0 + e1;
        pk[i] = pack_bf16x2(e0, e1);
      }
      l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      stamp(4 + 5 * j);
      tmem_st_32x32b_x32(tS, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_st_32x32b_x32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      stamp(5 + 5 * j);
    }
    stamp(kTraceSlots - 1);
    // epilogue: O / l -> global, lse
    if (ok && my_blk > 0) {
      ok = mbar_wait(&pv_done[t], (my_blk - 1) & 1, dead, p.status, 452);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool valid = qi < p.Sq;
      __nv_bfloat16* orow = (__nv_bfloat16*)p.out + (long)b * p.o_batch_stride + (long)qi * p.o_row_stride + (long)h * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (my_blk > 0) {
          tmem_ld_32x32b_x32(tO + c * 32, v);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
          }
        }
      }
      if (valid && p.lse)
        p.lse[((long)b * p.Hq + h) * p.Sq + qi] = l > 0.f ? (m * 0.6931471805599453f + logf(l)) : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc<kTmemCols>(tmem_base);
}

}  // namespace

namespace axh {
int make_bshd_map(CUtensorMap* m, const void* ptr, int D, int H, int S, int B, long row_stride,
                  long batch_stride, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)row_stride * 2, (uint64_t)batch_stride * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
}
}  // namespace axh

// Diagnostic timeline: the launches that follow stamp the softmax stage of two CTAs into `buf`
// ([2][128] 64-bit slots, zero-filled by the caller); null turns it off.
static unsigned long long* g_flash_trace = nullptr;
AX_API void ax_flash_fwd_set_trace(void* buf) { g_flash_trace = (unsigned long long*)buf; }
// 1: always run the kernel with one 128-query tile per CTA (for comparisons); 0: choose by length.
static int g_flash_one_tile = 0;
AX_API void ax_flash_fwd_set_one_tile(int flag) { g_flash_one_tile = flag; }

// q [B,Sq,Hq,128], k/v [B,Skv,Hkv,128], out [B,Sq,Hq,128] (bf16, token-major; strides in elements),
// lse [B,Hq,Sq] fp32.  Returns a cudaError_t value or a negative code for unsupported arguments.
AX_API int ax_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                        int Sq, int Skv, int Hq, int Hkv, int D, long q_row, long q_batch, long k_row,
                        long k_batch, long v_row, long v_batch, long o_row, long o_batch, int causal,
                        float scale, int* status, cudaStream_t stream) {
  if (D != fa::HD || Hq % Hkv != 0) return -1;
  if ((q_row | k_row | v_row | o_row | q_batch | k_batch | v_batch) % 8) return -1;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) return -1;
  if (B <= 0 || Sq <= 0 || Skv <= 0) return 0;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = axh::make_bshd_map(&mq, q, D, Hq, Sq, B, q_row, q_batch, BQ))) return 1000 + rc;
  if ((rc = axh::make_bshd_map(&mk, k, D, Hkv, Skv, B, k_row, k_batch, BKV))) return 2000 + rc;
  if ((rc = axh::make_bshd_map(&mv, v, D, Hkv, Skv, B, v_row, v_batch, BKV))) return 3000 + rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  FwdParams p;
  p.out = out; p.o_row_stride = o_row; p.o_batch_stride = o_batch; p.lse = lse;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv; p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.trace = g_flash_trace;
  if (Sq > BQ && g_flash_one_tile == 0) {
    // two query tiles per CTA
    static bool configured2 = false;
    if (!configured2) {
      cudaError_t e = cudaFuncSetAttribute(flash_fwd2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2);
      if (e != cudaSuccess) return (int)e;
      e = cudaFuncSetAttribute(flash_fwd2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2);
      if (e != cudaSuccess) return (int)e;
      configured2 = true;
    }
    dim3 grid2(((Sq + 2 * BQ - 1) / (2 * BQ)) * Hq * B, 1, 1);
    if (g_flash_trace != nullptr) flash_fwd2_kernel<true><<<grid2, kThreads2, kSmem2, stream>>>(mq, mk, mv, p);
    else flash_fwd2_kernel<false><<<grid2, kThreads2, kSmem2, stream>>>(mq, mk, mv, p);
    return (int)cudaGetLastError();
  }
  dim3 grid(((Sq + BQ - 1) / BQ) * Hq * B, 1, 1);
  flash_fwd_kernel<<<grid, kThreads, kSmem, stream>>>(mq, mk, mv, p);
  return (int)cudaGetLastError();
}
