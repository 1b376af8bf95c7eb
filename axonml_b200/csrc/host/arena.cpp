// Offset allocator for large device arenas (best fit, split on allocation, coalescing on free).
//
// The allocator never touches the memory it manages: it hands out byte offsets into a range
// [0, capacity).  Two users:
//   * the caching device allocator (core/storage.py): segments obtained once from the device are
//     carved into tensors here, so a training loop's allocate / free pattern costs no driver call;
//   * the symmetric heap (parallel/symm.py): one peer-mapped (and multicast-bound) arena per
//     process group, exchanged once; every rank makes the same calls in the same order, the
//     allocator is deterministic, so a sub-buffer has the same offset on every rank and its peer
//     and multicast addresses are base + offset without another exchange.
//
// The reference's allocator is a 64-byte aligned host allocation per tensor
// (crates/axonml-core/src/allocator.rs, backends/cpu.rs:64-82); it has no device pool.
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <utility>

#define AX_API extern "C" __attribute__((visibility("default")))

namespace {

struct Arena {
  uint64_t capacity, alignment;
  std::map<uint64_t, uint64_t> free_by_off;                  // offset -> size of every free block
  std::set<std::pair<uint64_t, uint64_t>> free_by_size;      // (size, offset): best fit = lower_bound
  std::map<uint64_t, uint64_t> used;                         // offset -> size of every live block
  uint64_t in_use = 0, peak = 0, allocations = 0;
  std::mutex mu;

  void add_free(uint64_t off, uint64_t size) {
    free_by_off[off] = size;
    free_by_size.insert({size, off});
  }
  void drop_free(uint64_t off, uint64_t size) {
    free_by_off.erase(off);
    free_by_size.erase({size, off});
  }
};

inline uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

}  // namespace

// capacity and alignment in bytes; alignment a power of two (0 -> 512).
AX_API void* ax_arena_create(uint64_t capacity, uint64_t alignment) {
  if (alignment == 0) alignment = 512;
  if (capacity == 0 || (alignment & (alignment - 1))) return nullptr;
  auto* a = new Arena();
  a->capacity = capacity / alignment * alignment;
  a->alignment = alignment;
  if (a->capacity == 0) { delete a; return nullptr; }
  a->add_free(0, a->capacity);
  return a;
}

AX_API void ax_arena_destroy(void* h) { delete static_cast<Arena*>(h); }

// Offset of a block of at least `bytes` bytes (a multiple of the alignment), or -1 when no free
// block is large enough.  Best fit; among equal sizes the lowest offset.
AX_API int64_t ax_arena_alloc(void* h, uint64_t bytes) {
  auto* a = static_cast<Arena*>(h);
  if (a == nullptr) return -1;
  std::lock_guard<std::mutex> g(a->mu);
  const uint64_t need = round_up(bytes == 0 ? 1 : bytes, a->alignment);
  auto it = a->free_by_size.lower_bound({need, 0});
  if (it == a->free_by_size.end()) return -1;
  const uint64_t size = it->first, off = it->second;
  a->drop_free(off, size);
  if (size > need) a->add_free(off + need, size - need);
  a->used[off] = need;
  a->in_use += need;
  if (a->in_use > a->peak) a->peak = a->in_use;
  ++a->allocations;
  return (int64_t)off;
}

// 0 on success, -1 when `offset` is not the start of a live block.
AX_API int ax_arena_free(void* h, int64_t offset) {
  auto* a = static_cast<Arena*>(h);
  if (a == nullptr || offset < 0) return -1;
  std::lock_guard<std::mutex> g(a->mu);
  auto u = a->used.find((uint64_t)offset);
  if (u == a->used.end()) return -1;
  uint64_t off = u->first, size = u->second;
  a->used.erase(u);
  a->in_use -= size;
  // merge with the free neighbours
  auto next = a->free_by_off.find(off + size);
  if (next != a->free_by_off.end()) {
    const uint64_t nsize = next->second;
    a->drop_free(off + size, nsize);
    size += nsize;
  }
  auto prev = a->free_by_off.lower_bound(off);
  if (prev != a->free_by_off.begin()) {
    --prev;
    if (prev->first + prev->second == off) {
      const uint64_t poff = prev->first, psize = prev->second;
      a->drop_free(poff, psize);
      off = poff;
      size += psize;
    }
  }
  a->add_free(off, size);
  return 0;
}

// Size of the live block at `offset`, or 0.
AX_API uint64_t ax_arena_block_size(void* h, int64_t offset) {
  auto* a = static_cast<Arena*>(h);
  if (a == nullptr || offset < 0) return 0;
  std::lock_guard<std::mutex> g(a->mu);
  auto u = a->used.find((uint64_t)offset);
  return u == a->used.end() ? 0 : u->second;
}

// out[0..6] = capacity, bytes in use, peak bytes in use, live blocks, free blocks, largest free
// block, allocations made so far.
AX_API void ax_arena_stats(void* h, uint64_t* out) {
  auto* a = static_cast<Arena*>(h);
  if (a == nullptr) return;
  std::lock_guard<std::mutex> g(a->mu);
  out[0] = a->capacity;
  out[1] = a->in_use;
  out[2] = a->peak;
  out[3] = a->used.size();
  out[4] = a->free_by_off.size();
  out[5] = a->free_by_size.empty() ? 0 : a->free_by_size.rbegin()->first;
  out[6] = a->allocations;
}

// Frees every block (the peak and the allocation count are kept).
AX_API void ax_arena_reset(void* h) {
  auto* a = static_cast<Arena*>(h);
  if (a == nullptr) return;
  std::lock_guard<std::mutex> g(a->mu);
  a->free_by_off.clear();
  a->free_by_size.clear();
  a->used.clear();
  a->in_use = 0;
  a->add_free(0, a->capacity);
}
