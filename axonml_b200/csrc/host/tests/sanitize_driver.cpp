// Exercises the host library on exactly-sized heap buffers so that AddressSanitizer and
// UndefinedBehaviorSanitizer see any overrun, misaligned access or overflow.  Built and run by
// tests/test_host_sanitizers.py with -fsanitize=address,undefined -fno-sanitize-recover=all; it is
// not part of the shipped library.  The reference has no sanitizer jobs (its CI is check / test /
// fmt / clippy).
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

extern "C" {
int ax_quant_block_elems(int type);
int ax_quant_block_bytes(int type);
int ax_quantize(int type, int layout, const float* x, uint8_t* out, int64_t n);
int ax_dequantize(int type, int layout, const uint8_t* in, float* y, int64_t n);
void ax_f32_to_f16(const float* x, uint16_t* y, int64_t n);
void ax_f16_to_f32(const uint16_t* x, float* y, int64_t n);
void* ax_bc_writer_new();
void ax_bc_writer_free(void* w);
void ax_bc_write_u64(void* w, uint64_t v);
void ax_bc_write_str(void* w, const char* s, uint64_t n);
void ax_bc_write_entry(void* w, const uint64_t* shape, uint64_t ndim, const float* vals, uint64_t nvals, uint8_t rg);
uint64_t ax_bc_writer_size(void* w);
const uint8_t* ax_bc_writer_data(void* w);
void* ax_bc_open_state_dict(const uint8_t* data, uint64_t len, uint64_t start);
void ax_bc_close(void* r);
uint64_t ax_bc_count(void* r);
int ax_bc_entry(void* r, uint64_t i, uint64_t* out);
void ax_cpu_binary(int op, const float* a, const float* b, float* y, int64_t n);
void ax_cpu_unary(int op, const float* x, float* y, int64_t n, float p);
double ax_cpu_reduce(int op, const float* x, int64_t n);
void ax_cpu_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K);
void ax_cpu_transpose(const float* x, float* y, int64_t rows, int64_t cols);
void ax_cpu_softmax_rows(const float* x, float* y, int64_t rows, int64_t cols, int log_mode);
void ax_cpu_embedding(const int64_t* idx, const float* W, float* y, int64_t n, int64_t D, int64_t V);
}

static int fails = 0;
#define CHECK(c)                                                      \
  do {                                                                \
    if (!(c)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #c); ++fails; } \
  } while (0)

static float* heap_f(int64_t n, unsigned seed) {      // exactly n floats, no slack
  float* p = (float*)std::malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
  for (int64_t i = 0; i < n; ++i) { seed = seed * 1664525u + 1013904223u; p[i] = ((int)(seed >> 9) % 2001 - 1000) / 250.f; }
  return p;
}

static void quant_roundtrips() {
  for (int type = 0; type < 6; ++type) {
    const int be = ax_quant_block_elems(type), bb = ax_quant_block_bytes(type);
    for (int layout = 0; layout < 2; ++layout) {
      if (layout == 1 && (type == 0 || type == 3 || type == 4)) continue;   // adjacent pairs: 4-bit formats
      for (int blocks : {1, 3, 17}) {
        const int64_t n = (int64_t)blocks * be;
        float* x = heap_f(n, 7u + type);
        uint8_t* q = (uint8_t*)std::malloc((size_t)blocks * bb);
        float* y = (float*)std::malloc((size_t)n * sizeof(float));
        CHECK(ax_quantize(type, layout, x, q, n) == 0);
        CHECK(ax_dequantize(type, layout, q, y, n) == 0);
        double err = 0, ref = 0;
        for (int64_t i = 0; i < n; ++i) { err += std::fabs(x[i] - y[i]); ref += std::fabs(x[i]); }
        CHECK(err <= 0.2 * ref + 1e-6);
        CHECK(ax_quantize(type, layout, x, q, n - 1) != 0);                 // ragged length is refused, nothing written
        std::free(x); std::free(q); std::free(y);
      }
    }
  }
  const int64_t n = 33;
  float* x = heap_f(n, 3u);
  uint16_t* h = (uint16_t*)std::malloc(n * 2);
  float* y = (float*)std::malloc(n * 4);
  ax_f32_to_f16(x, h, n);
  ax_f16_to_f32(h, y, n);
  for (int64_t i = 0; i < n; ++i) CHECK(std::fabs(x[i] - y[i]) <= 4e-3f * (1.f + std::fabs(x[i])));
  std::free(x); std::free(h); std::free(y);
}

static void bincode_roundtrip_and_truncation() {
  void* w = ax_bc_writer_new();
  ax_bc_write_u64(w, 2);                                   // two entries
  const uint64_t shape_a[2] = {3, 5};
  float* a = heap_f(15, 11u);
  ax_bc_write_str(w, "layer.weight", 12);
  ax_bc_write_entry(w, shape_a, 2, a, 15, 1);
  ax_bc_write_u64(w, 0);                                   // entry metadata: empty map
  const uint64_t shape_b[1] = {7};
  float* b = heap_f(7, 12u);
  ax_bc_write_str(w, "layer.bias", 10);
  ax_bc_write_entry(w, shape_b, 1, b, 7, 0);
  ax_bc_write_u64(w, 0);
  ax_bc_write_u64(w, 0);                                   // state-dict metadata: empty map
  const uint64_t len = ax_bc_writer_size(w);
  uint8_t* exact = (uint8_t*)std::malloc(len);             // the reader gets a buffer with no slack
  std::memcpy(exact, ax_bc_writer_data(w), len);
  void* r = ax_bc_open_state_dict(exact, len, 0);
  CHECK(r != nullptr);
  if (r) {
    CHECK(ax_bc_count(r) == 2);
    uint64_t e[9];
    CHECK(ax_bc_entry(r, 0, e) == 0 && e[1] == 12 && e[2] == 2 && e[4] == 15 && e[6] == 1);
    CHECK(std::memcmp(exact + e[5], a, 15 * 4) == 0);
    CHECK(ax_bc_entry(r, 1, e) == 0 && e[1] == 10 && e[4] == 7 && e[6] == 0);
    CHECK(ax_bc_entry(r, 2, e) != 0);
    ax_bc_close(r);
  }
  // every truncation of the stream must be refused without reading past the end
  for (uint64_t cut = 0; cut < len; ++cut) {
    uint8_t* t = (uint8_t*)std::malloc(cut ? cut : 1);
    std::memcpy(t, exact, cut);
    void* rr = ax_bc_open_state_dict(t, cut, 0);
    CHECK(rr == nullptr);
    if (rr) ax_bc_close(rr);
    std::free(t);
  }
  // hostile counts (a length field of 2^63) must be refused, not allocated or walked
  uint8_t* evil = (uint8_t*)std::malloc(len);
  std::memcpy(evil, exact, len);
  std::memset(evil + 8, 0xff, 7);                          // key length of entry 0
  void* re = ax_bc_open_state_dict(evil, len, 0);
  CHECK(re == nullptr);
  if (re) ax_bc_close(re);
  std::free(evil); std::free(exact); std::free(a); std::free(b);
  ax_bc_writer_free(w);
}

static void cpu_kernels_ragged_sizes() {
  for (int64_t n : {1, 7, 16, 33, 257}) {
    float *a = heap_f(n, 21u), *b = heap_f(n, 22u);
    float* y = (float*)std::malloc((size_t)n * 4);
    for (int op = 0; op < 4; ++op) ax_cpu_binary(op, a, b, y, n);
    for (int op = 0; op < 8; ++op) ax_cpu_unary(op, a, y, n, 0.1f);
    double s = ax_cpu_reduce(0, a, n), ref = 0;
    for (int64_t i = 0; i < n; ++i) ref += a[i];
    CHECK(std::fabs(s - ref) < 1e-3 * (1 + std::fabs(ref)));
    std::free(a); std::free(b); std::free(y);
  }
  const int64_t M = 5, N = 7, K = 3;
  float *A = heap_f(M * K, 31u), *B = heap_f(K * N, 32u);
  float* C = (float*)std::malloc(M * N * 4);
  ax_cpu_matmul(A, B, C, M, N, K);
  double ref = 0;
  for (int64_t k = 0; k < K; ++k) ref += (double)A[2 * K + k] * B[k * N + 4];
  CHECK(std::fabs(C[2 * N + 4] - ref) < 1e-4);
  float* T = (float*)std::malloc(M * N * 4);
  ax_cpu_transpose(C, T, M, N);
  CHECK(T[4 * M + 2] == C[2 * N + 4]);
  float* S = (float*)std::malloc(M * N * 4);
  ax_cpu_softmax_rows(C, S, M, N, 0);
  double rs = 0;
  for (int64_t j = 0; j < N; ++j) rs += S[3 * N + j];
  CHECK(std::fabs(rs - 1.0) < 1e-5);
  const int64_t V = 4, D = 3;
  float* W = heap_f(V * D, 41u);
  int64_t idx[5] = {0, 3, 1, 3, 2};
  float* E = (float*)std::malloc(5 * D * 4);
  ax_cpu_embedding(idx, W, E, 5, D, V);
  CHECK(E[1 * D + 2] == W[3 * D + 2]);
  std::free(A); std::free(B); std::free(C); std::free(T); std::free(S); std::free(W); std::free(E);
}

int main() {
  quant_roundtrips();
  bincode_roundtrip_and_truncation();
  cpu_kernels_ragged_sizes();
  std::printf(fails ? "sanitize_driver: %d failure(s)\n" : "sanitize_driver: ok\n", fails);
  return fails ? 1 : 0;
}
