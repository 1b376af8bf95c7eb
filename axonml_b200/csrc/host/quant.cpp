// Block quantisation codecs on the CPU (OpenMP): Q8_0, Q4_0, Q4_1, Q5_0, Q5_1 (32-element blocks)
// and Q4_K (256-element super-blocks), in the GGML/GGUF byte layouts, plus the reference's own
// adjacent-pair nibble order for Q4_0/Q4_1 (crates/axonml-quant/src/types.rs:179-198).
//
// Formulas of the 32-element formats follow crates/axonml-quant/src/quantize.rs:82-205
// (Q8_0: scale = absmax/127; Q4_0: scale = absmax/7, values clamped to [-8,7]; Q4_1: scale =
// (max-min)/15 with a stored minimum).  Q5_0/Q5_1 are real 5-bit codecs here (the reference falls
// back to Q4_0, quantize.rs:47-50).  Q4_K: 8 sub-blocks of 32, 6-bit sub-scales and sub-minimums
// packed in 12 bytes, fp16 super-scale d and dmin, 128 bytes of nibbles = 144 bytes.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>

#define AX_API extern "C" __attribute__((visibility("default")))

namespace {

// ---- fp16 <-> fp32 (round to nearest even), no hardware dependency
inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    int shift = 14 - exp;
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = (uint32_t)(exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
  return (uint16_t)(sign | half);
}
inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) x = sign;
    else {
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      x = sign | (uint32_t)((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    x = sign | 0x7f800000u | (man << 13);
  } else {
    x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &x, 4);
  return f;
}

constexpr int QK = 32;
constexpr int QK_K = 256;

inline int nearest(float v) { return (int)lrintf(v); }

// Q4_K helper: pick scale and min for 32 values so that x ~ scale*q - min, q in [0, 15]
float make_qkx(const float* x, int n, int nmax, uint8_t* L, float* the_min) {
  float mn = x[0], mx = x[0];
  for (int i = 1; i < n; ++i) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
  if (mn > 0) mn = 0;
  if (mx <= mn) {
    for (int i = 0; i < n; ++i) L[i] = 0;
    *the_min = -mn;
    return 0.f;
  }
  float iscale = nmax / (mx - mn), scale = 1.f / iscale;
  // a few refinement rounds: re-fit scale/min to the rounded codes (least squares)
  for (int it = 0; it < 4; ++it) {
    double sl = 0, sl2 = 0, sx = 0, sxl = 0;
    for (int i = 0; i < n; ++i) {
      int l = std::max(0, std::min(nmax, nearest(iscale * (x[i] - mn))));
      L[i] = (uint8_t)l;
      sl += l; sl2 += (double)l * l; sx += x[i]; sxl += (double)x[i] * l;
    }
    double D = n * sl2 - sl * sl;
    if (D <= 0) break;
    double s = (n * sxl - sx * sl) / D, m = (sl2 * sx - sl * sxl) / D;
    if (s <= 0) break;
    if (m > 0) { m = 0; s = sl2 > 0 ? sxl / sl2 : s; }
    scale = (float)s; mn = (float)m; iscale = 1.f / scale;
  }
  for (int i = 0; i < n; ++i) L[i] = (uint8_t)std::max(0, std::min(nmax, nearest(iscale * (x[i] - mn))));
  *the_min = -mn;
  return scale;
}

inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
  else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

}  // namespace

// type ids: 0 Q8_0 (34 B), 1 Q4_0 (18 B), 2 Q4_1 (20 B), 3 Q5_0 (22 B), 4 Q5_1 (24 B), 5 Q4_K (144 B / 256)
AX_API int ax_quant_block_elems(int type) { return type == 5 ? QK_K : QK; }
AX_API int ax_quant_block_bytes(int type) {
  static const int b[6] = {34, 18, 20, 22, 24, 144};
  return (type >= 0 && type < 6) ? b[type] : -1;
}

// n must be a multiple of the block size.  layout: 0 = GGML nibble order (element j and j+16 share
// a byte), 1 = adjacent pairs (elements 2i, 2i+1 share a byte; 4-bit formats only).
AX_API int ax_quantize(int type, int layout, const float* x, uint8_t* out, int64_t n) {
  const int be = ax_quant_block_elems(type), bb = ax_quant_block_bytes(type);
  if (bb < 0 || n % be) return -1;
  const int64_t nb = n / be;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; ++b) {
    const float* v = x + b * be;
    uint8_t* o = out + b * bb;
    if (type == 0) {
      float amax = 0;
      for (int i = 0; i < QK; ++i) amax = std::max(amax, std::fabs(v[i]));
      float d = amax / 127.f, id = d ? 1.f / d : 0.f;
      uint16_t h = f32_to_f16(d);
      memcpy(o, &h, 2);
      for (int i = 0; i < QK; ++i) ((int8_t*)(o + 2))[i] = (int8_t)std::max(-127, std::min(127, nearest(v[i] * id)));
    } else if (type == 1 || type == 2) {
      float mn = v[0], mx = v[0], amax = 0;
      for (int i = 0; i < QK; ++i) { mn = std::min(mn, v[i]); mx = std::max(mx, v[i]); amax = std::max(amax, std::fabs(v[i])); }
      float d, id, base;
      int hdr;
      if (type == 1) { d = amax / 7.f; base = 0; hdr = 2; }
      else { d = (mx - mn) / 15.f; base = mn; hdr = 4; uint16_t hm = f32_to_f16(mn); memcpy(o + 2, &hm, 2); }
      id = d ? 1.f / d : 0.f;
      uint16_t h = f32_to_f16(d);
      memcpy(o, &h, 2);
      uint8_t q[QK];
      for (int i = 0; i < QK; ++i) {
        if (type == 1) q[i] = (uint8_t)(std::max(-8, std::min(7, nearest(v[i] * id))) + 8);
        else q[i] = (uint8_t)std::max(0, std::min(15, nearest((v[i] - base) * id)));
      }
      for (int i = 0; i < 16; ++i)
        o[hdr + i] = layout == 1 ? (uint8_t)(q[2 * i] | (q[2 * i + 1] << 4)) : (uint8_t)(q[i] | (q[i + 16] << 4));
    } else if (type == 3 || type == 4) {
      float mn = v[0], mx = v[0], amax = 0;
      for (int i = 0; i < QK; ++i) { mn = std::min(mn, v[i]); mx = std::max(mx, v[i]); amax = std::max(amax, std::fabs(v[i])); }
      float d, id, base;
      int hdr;
      if (type == 3) { d = amax / 15.f; base = 0; hdr = 2; }
      else { d = (mx - mn) / 31.f; base = mn; hdr = 4; uint16_t hm = f32_to_f16(mn); memcpy(o + 2, &hm, 2); }
      id = d ? 1.f / d : 0.f;
      uint16_t h = f32_to_f16(d);
      memcpy(o, &h, 2);
      uint32_t qh = 0;
      uint8_t q[QK];
      for (int i = 0; i < QK; ++i) {
        if (type == 3) q[i] = (uint8_t)(std::max(-16, std::min(15, nearest(v[i] * id))) + 16);
        else q[i] = (uint8_t)std::max(0, std::min(31, nearest((v[i] - base) * id)));
      }
      for (int i = 0; i < 16; ++i) {
        o[hdr + 4 + i] = (uint8_t)((q[i] & 0xF) | ((q[i + 16] & 0xF) << 4));
        qh |= (uint32_t)((q[i] >> 4) & 1) << i;
        qh |= (uint32_t)((q[i + 16] >> 4) & 1) << (i + 16);
      }
      memcpy(o + hdr, &qh, 4);
    } else {  // Q4_K
      uint8_t L[QK_K];
      float scales[8], mins[8];
      float max_scale = 0, max_min = 0;
      for (int j = 0; j < 8; ++j) {
        scales[j] = make_qkx(v + 32 * j, 32, 15, L + 32 * j, &mins[j]);
        max_scale = std::max(max_scale, scales[j]);
        max_min = std::max(max_min, mins[j]);
      }
      float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f, inv_min = max_min > 0 ? 63.f / max_min : 0.f;
      uint8_t* sc = o + 4;
      memset(sc, 0, 12);
      for (int j = 0; j < 8; ++j) {
        uint8_t ls = (uint8_t)std::min(63, nearest(inv_scale * scales[j]));
        uint8_t lm = (uint8_t)std::min(63, nearest(inv_min * mins[j]));
        if (j < 4) { sc[j] = ls; sc[j + 4] = lm; }
        else { sc[j + 4] = (ls & 0xF) | ((lm & 0xF) << 4); sc[j - 4] |= (ls >> 4) << 6; sc[j] |= (lm >> 4) << 6; }
      }
      uint16_t hd = f32_to_f16(max_scale / 63.f), hm = f32_to_f16(max_min / 63.f);
      memcpy(o, &hd, 2);
      memcpy(o + 2, &hm, 2);
      const float dd = f16_to_f32(hd), dm = f16_to_f32(hm);
      for (int j = 0; j < 8; ++j) {
        uint8_t s6, m6;
        get_scale_min_k4(j, sc, &s6, &m6);
        float d = dd * s6, m = dm * m6;
        if (d == 0) { for (int i = 0; i < 32; ++i) L[32 * j + i] = 0; continue; }
        for (int i = 0; i < 32; ++i)
          L[32 * j + i] = (uint8_t)std::max(0, std::min(15, nearest((v[32 * j + i] + m) / d)));
      }
      uint8_t* q = o + 16;
      for (int j = 0; j < QK_K; j += 64)
        for (int l = 0; l < 32; ++l) *q++ = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
    }
  }
  return 0;
}

AX_API int ax_dequantize(int type, int layout, const uint8_t* in, float* y, int64_t n) {
  const int be = ax_quant_block_elems(type), bb = ax_quant_block_bytes(type);
  if (bb < 0 || n % be) return -1;
  const int64_t nb = n / be;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; ++b) {
    const uint8_t* o = in + b * bb;
    float* v = y + b * be;
    uint16_t h;
    memcpy(&h, o, 2);
    const float d = f16_to_f32(h);
    if (type == 0) {
      for (int i = 0; i < QK; ++i) v[i] = d * ((const int8_t*)(o + 2))[i];
    } else if (type == 1 || type == 2) {
      float m = 0;
      int hdr = 2;
      if (type == 2) { uint16_t hm; memcpy(&hm, o + 2, 2); m = f16_to_f32(hm); hdr = 4; }
      for (int i = 0; i < 16; ++i) {
        int lo = o[hdr + i] & 0xF, hi = o[hdr + i] >> 4;
        int i0 = layout == 1 ? 2 * i : i, i1 = layout == 1 ? 2 * i + 1 : i + 16;
        v[i0] = type == 1 ? d * (lo - 8) : d * lo + m;
        v[i1] = type == 1 ? d * (hi - 8) : d * hi + m;
      }
    } else if (type == 3 || type == 4) {
      float m = 0;
      int hdr = 2;
      if (type == 4) { uint16_t hm; memcpy(&hm, o + 2, 2); m = f16_to_f32(hm); hdr = 4; }
      uint32_t qh;
      memcpy(&qh, o + hdr, 4);
      for (int i = 0; i < 16; ++i) {
        int lo = (o[hdr + 4 + i] & 0xF) | (((qh >> i) & 1) << 4);
        int hi = (o[hdr + 4 + i] >> 4) | (((qh >> (i + 16)) & 1) << 4);
        v[i] = type == 3 ? d * (lo - 16) : d * lo + m;
        v[i + 16] = type == 3 ? d * (hi - 16) : d * hi + m;
      }
    } else {
      uint16_t hm;
      memcpy(&hm, o + 2, 2);
      const float dmin = f16_to_f32(hm);
      const uint8_t* sc = o + 4;
      const uint8_t* q = o + 16;
      int is = 0;
      for (int j = 0; j < QK_K; j += 64) {
        uint8_t s, mm;
        get_scale_min_k4(is, sc, &s, &mm);
        const float d1 = d * s, m1 = dmin * mm;
        get_scale_min_k4(is + 1, sc, &s, &mm);
        const float d2 = d * s, m2 = dmin * mm;
        for (int l = 0; l < 32; ++l) v[j + l] = d1 * (q[l] & 0xF) - m1;
        for (int l = 0; l < 32; ++l) v[j + 32 + l] = d2 * (q[l] >> 4) - m2;
        q += 32;
        is += 2;
      }
    }
  }
  return 0;
}

AX_API void ax_f32_to_f16(const float* x, uint16_t* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = f32_to_f16(x[i]);
}
AX_API void ax_f16_to_f32(const uint16_t* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = f16_to_f32(x[i]);
}
