// bincode-1.x (little-endian, fixed-width integers, u64 lengths) codec for the reference's
// checkpoint containers (crates/axonml-serialize/src/state_dict.rs:16-99, checkpoint.rs:16-137):
//
//   StateDict  = map<String, StateDictEntry>, map<String,String>
//   Entry      = TensorData{shape: Vec<usize>, values: Vec<f32>}, requires_grad: bool,
//                metadata: map<String,String>
//
// The reader builds an index over an in-memory file (offsets of every key, shape and value run)
// so that Python can wrap the float payloads without copying; the writer appends to a growable
// buffer.  Both are plain C entry points used through ctypes.
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#define AX_API extern "C" __attribute__((visibility("default")))

namespace {

struct Writer {
  std::vector<uint8_t> buf;
  void u64(uint64_t v) { put(&v, 8); }
  void u8(uint8_t v) { buf.push_back(v); }
  void put(const void* p, size_t n) {
    const uint8_t* b = (const uint8_t*)p;
    buf.insert(buf.end(), b, b + n);
  }
  void str(const char* s, uint64_t n) { u64(n); put(s, n); }
};

struct Entry {
  uint64_t key_off, key_len;
  uint64_t ndim, shape_off;
  uint64_t nvals, data_off;
  uint8_t requires_grad;
  uint64_t nmeta, meta_off;     // meta_off: offset of the first (klen,k,vlen,v) pair
};

struct Reader {
  const uint8_t* p = nullptr;
  uint64_t len = 0, pos = 0;
  bool ok = true;
  std::vector<Entry> entries;
  uint64_t nmeta = 0, meta_off = 0;   // state-dict level metadata
  uint64_t end = 0;                   // offset just after the StateDict

  uint64_t u64() {
    if (pos + 8 > len) { ok = false; return 0; }
    uint64_t v;
    memcpy(&v, p + pos, 8);
    pos += 8;
    return v;
  }
  uint8_t u8() {
    if (pos + 1 > len) { ok = false; return 0; }
    return p[pos++];
  }
  bool skip(uint64_t n) {
    if (n > len || pos + n > len) { ok = false; return false; }
    pos += n;
    return true;
  }
  bool skip_str() { uint64_t n = u64(); return ok && skip(n); }
  bool skip_map() {
    uint64_t n = u64();
    for (uint64_t i = 0; ok && i < n; ++i) { skip_str(); skip_str(); }
    return ok;
  }
  bool parse_state_dict() {
    uint64_t n = u64();
    if (!ok || n > (1ull << 32)) { ok = false; return false; }
    entries.reserve(n);
    for (uint64_t i = 0; ok && i < n; ++i) {
      Entry e{};
      e.key_len = u64();
      e.key_off = pos;
      if (!skip(e.key_len)) break;
      e.ndim = u64();
      e.shape_off = pos;
      if (e.ndim > 64 || !skip(e.ndim * 8)) { ok = false; break; }
      e.nvals = u64();
      e.data_off = pos;
      if (e.nvals > (1ull << 40) || !skip(e.nvals * 4)) { ok = false; break; }
      e.requires_grad = u8();
      e.nmeta = u64();
      e.meta_off = pos;
      for (uint64_t m = 0; ok && m < e.nmeta; ++m) { skip_str(); skip_str(); }
      entries.push_back(e);
    }
    nmeta = u64();
    meta_off = pos;
    for (uint64_t m = 0; ok && m < nmeta; ++m) { skip_str(); skip_str(); }
    end = pos;
    return ok;
  }
};

}  // namespace

// ------------------------------------------------------------------ writer
AX_API void* ax_bc_writer_new() { return new Writer(); }
AX_API void ax_bc_writer_free(void* w) { delete (Writer*)w; }
AX_API void ax_bc_write_u64(void* w, uint64_t v) { ((Writer*)w)->u64(v); }
AX_API void ax_bc_write_u8(void* w, uint8_t v) { ((Writer*)w)->u8(v); }
AX_API void ax_bc_write_f32(void* w, float v) { ((Writer*)w)->put(&v, 4); }
AX_API void ax_bc_write_str(void* w, const char* s, uint64_t n) { ((Writer*)w)->str(s, n); }
AX_API void ax_bc_write_raw(void* w, const void* p, uint64_t n) { ((Writer*)w)->put(p, n); }
// one StateDictEntry body (after its key): tensor data, requires_grad, empty or given metadata
AX_API void ax_bc_write_entry(void* w, const uint64_t* shape, uint64_t ndim, const float* vals,
                              uint64_t nvals, uint8_t requires_grad) {
  Writer* W = (Writer*)w;
  W->u64(ndim);
  W->put(shape, ndim * 8);
  W->u64(nvals);
  W->put(vals, nvals * 4);
  W->u8(requires_grad);
}
AX_API uint64_t ax_bc_writer_size(void* w) { return ((Writer*)w)->buf.size(); }
AX_API const uint8_t* ax_bc_writer_data(void* w) { return ((Writer*)w)->buf.data(); }

// ------------------------------------------------------------------ reader
// Parses a StateDict that starts at `start` inside [data, data+len).  Returns a handle or null.
AX_API void* ax_bc_open_state_dict(const uint8_t* data, uint64_t len, uint64_t start) {
  Reader* r = new Reader();
  r->p = data; r->len = len; r->pos = start;
  if (!r->parse_state_dict()) { delete r; return nullptr; }
  return r;
}
AX_API void ax_bc_close(void* r) { delete (Reader*)r; }
AX_API uint64_t ax_bc_count(void* r) { return ((Reader*)r)->entries.size(); }
AX_API uint64_t ax_bc_end(void* r) { return ((Reader*)r)->end; }
AX_API uint64_t ax_bc_meta_count(void* r) { return ((Reader*)r)->nmeta; }
AX_API uint64_t ax_bc_meta_offset(void* r) { return ((Reader*)r)->meta_off; }
// out[0..8] = key_off, key_len, ndim, shape_off, nvals, data_off, requires_grad, nmeta, meta_off
AX_API int ax_bc_entry(void* r, uint64_t i, uint64_t* out) {
  Reader* R = (Reader*)r;
  if (i >= R->entries.size()) return -1;
  const Entry& e = R->entries[i];
  out[0] = e.key_off; out[1] = e.key_len; out[2] = e.ndim; out[3] = e.shape_off; out[4] = e.nvals;
  out[5] = e.data_off; out[6] = e.requires_grad; out[7] = e.nmeta; out[8] = e.meta_off;
  return 0;
}
