// Shared pieces of the flash-attention kernels (forward, dQ, dK/dV): tensor maps over the
// token-major [B, S, H, D] layout, shared-memory tile conventions, and the tcgen05 operand
// descriptors for 128x128 / 128x64 bf16 tiles with head_dim 128.
//
// Tile convention: a [rows x 128] bf16 tile is kept as two "slabs" of [rows x 64] (one 128-byte
// swizzled row per tile row); slab h holds columns [64h, 64h+64).  The same bytes serve
//   * as a K-major operand   (reduction over the 128 columns):  8 MMAs, step k -> slab k/4,
//     +32 bytes per step inside the slab;
//   * as an MN-major operand (reduction over the rows, the 128 columns are the N/M extent):
//     +2048 bytes per 16 rows, slabs `rows*128` bytes apart (the descriptor's leading offset).
#pragma once
#include "common.cuh"

namespace fa {
using namespace ax;

constexpr int HD = 128;          // head dim handled by these kernels
constexpr int kSlabCols = 64;

struct TensorDesc4 {             // one of q / k / v / o / do ... as [B, S, H, D]
  const void* ptr;
  long row_stride;               // elements between consecutive tokens
  long batch_stride;             // elements between batches
  int heads;
  int seq;
  int batch;
};

__device__ __forceinline__ uint32_t slab_bytes(int rows) { return (uint32_t)rows * 128u; }

// K-major descriptor for MMA k-step `k` (16 columns) of a [rows x 128] tile.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int rows, int k) {
  return umma_desc_sw128(tile + (uint32_t)(k >> 2) * slab_bytes(rows) + (uint32_t)(k & 3) * 32u, 16,
                         1024);
}
// MN-major descriptor for MMA k-step `k` (16 rows) of a [rows x 128] tile (N/M = the 128 columns).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int rows, int k) {
  return umma_desc_sw128(tile + (uint32_t)k * 2048u, slab_bytes(rows), 1024);
}

// Stores 8 consecutive bf16 (one 16-byte chunk, chunk index c in [0,16)) of row r of a
// [rows x 128] tile held as two swizzled slabs.
__device__ __forceinline__ void store_tile_chunk(uint8_t* tile, int rows, int r, int c, uint4 v) {
  uint8_t* slab = tile + (c >> 3) * slab_bytes(rows);
  *reinterpret_cast<uint4*>(slab + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
}

}  // namespace fa

namespace axh {
// 4-D tensor map over a token-major [B, S, H, D] bf16 tensor; box = [1, box_rows, 1, 64].
int make_bshd_map(CUtensorMap* m, const void* ptr, int D, int H, int S, int B, long row_stride,
                  long batch_stride, int box_rows);
}
