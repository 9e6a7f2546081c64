/*
 * CPU oracle for the GGUF quantized-linear path. TEST INFRASTRUCTURE ONLY: linked by the
 * tests, the smoke check and the benchmark's CPU-baseline leg, never by the CUDA library.
 *
 * Restates (in plain C) what tur obtains from candle-core 0.10.2 (Cargo.lock:316-320,
 * source not vendored in the reference tree) at these call sites:
 *   QTensor::dequantize   src/weights/mod.rs:150,161; src/models/layers/mod.rs:37;
 *                         src/models/layers/norm.rs:82-84; src/models/layers/linear.rs:66
 *   QMatMul::forward      src/models/layers/linear.rs:24
 * Block layouts follow the GGUF wire format as documented by the `gguf` 0.19.0 python
 * package (quants.py: Q8_0 378-401, Q4_K 475-522, Q5_K 525-549, Q6_K 552-572;
 * constants.py GGML_QUANT_SIZES).
 *
 * Pinned bit-exact against that package: dequantize of all four weight types and the
 * Q8_0 quantizer. PARITY UNPINNED against candle itself: the Q8_K activation quantizer
 * (candle-core's published quantizer restated: iscale = -128/max, ties away from zero, clamp
 * to 127; divisor, scale sign and rounding are the compile-time switches TQO_Q8K_*),
 * the K-quant weight quantizers (own deterministic min/max + least-squares search; they
 * only have to emit valid blocks) and the f32 summation order of the block dots.
 */
#include "turq_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK8_0 32
#define QK_K 256

/* ------------------------------------------------------------------ scalar conversions */

float tqo_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t tqo_f32_to_f16(float f) { /* round to nearest even, IEEE semantics */
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | (absx > 0x7F800000u ? 0x200u | ((absx >> 13) & 0x3FFu) : 0));
  }
  if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 -> inf */
  if (absx < 0x33000001u) return (uint16_t)sign;              /* < 2^-25 (or == 2^-25 tie -> 0) */
  int32_t e = (int32_t)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) { /* subnormal result */
    shift = 13 + (-14 - e);
    base = 0;
  } else {
    shift = 13;
    base = ((uint32_t)(e + 15) << 10) - 0x400u; /* implicit bit is added back by man>>13 */
  }
  uint32_t q = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  return (uint16_t)(sign | (base + q));
}

float tqo_bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t tqo_f32_to_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  x += 0x7FFFu + ((x >> 16) & 1u);
  return (uint16_t)(x >> 16);
}

/* ------------------------------------------------------------------ block geometry */

int tqo_block_elems(int dtype) {
  switch (dtype) {
    case TQO_Q8_0: return QK8_0;
    case TQO_Q4_K: case TQO_Q5_K: case TQO_Q6_K: case TQO_Q8_K: return QK_K;
    case TQO_F32: case TQO_F16: case TQO_BF16: return 1;
    default: return 0;
  }
}

int tqo_block_bytes(int dtype) {
  switch (dtype) {
    case TQO_Q8_0: return 34;
    case TQO_Q4_K: return 144;
    case TQO_Q5_K: return 176;
    case TQO_Q6_K: return 210;
    case TQO_Q8_K: return 292;
    case TQO_F32: return 4;
    case TQO_F16: case TQO_BF16: return 2;
    default: return 0;
  }
}

size_t tqo_row_bytes(int dtype, int64_t k) {
  int be = tqo_block_elems(dtype);
  if (be == 0 || k < 0 || k % be != 0) return 0;
  return (size_t)(k / be) * (size_t)tqo_block_bytes(dtype);
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline void wr16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)(v & 0xFF); p[1] = (uint8_t)(v >> 8); }

/* 6-bit scale/min unpacking shared by Q4_K and Q5_K (12 bytes -> 8 scales + 8 mins),
 * gguf quants.py:479-500 */
static inline void k4_scale_min(const uint8_t* s, int j, int* sc, int* m) {
  if (j < 4) {
    *sc = s[j] & 63;
    *m = s[j + 4] & 63;
  } else {
    *sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
    *m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
  }
}

static inline void k4_pack_scale_min(uint8_t* s, const int* sc, const int* m) {
  memset(s, 0, 12);
  for (int j = 0; j < 8; j++) {
    if (j < 4) {
      s[j] = (uint8_t)sc[j];
      s[j + 4] = (uint8_t)m[j];
    } else {
      s[j + 4] = (uint8_t)((sc[j] & 0x0F) | ((m[j] & 0x0F) << 4));
      s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
      s[j] |= (uint8_t)((m[j] >> 4) << 6);
    }
  }
}

/* ------------------------------------------------------------------ integer unpacking
 * Each helper expands one block's quants to int8 q[elements] in element order. */

static void unpack_q4k(const uint8_t* b, int8_t* q) { /* b -> block start */
  const uint8_t* qs = b + 16;
  for (int g = 0; g < 4; g++)
    for (int i = 0; i < 32; i++) {
      q[64 * g + i] = (int8_t)(qs[32 * g + i] & 0x0F);
      q[64 * g + 32 + i] = (int8_t)(qs[32 * g + i] >> 4);
    }
}

static void unpack_q5k(const uint8_t* b, int8_t* q) {
  const uint8_t* qh = b + 16;
  const uint8_t* qs = b + 48;
  for (int g = 0; g < 4; g++)
    for (int i = 0; i < 32; i++) {
      q[64 * g + i] = (int8_t)((qs[32 * g + i] & 0x0F) | (((qh[i] >> (2 * g)) & 1) << 4));
      q[64 * g + 32 + i] = (int8_t)((qs[32 * g + i] >> 4) | (((qh[i] >> (2 * g + 1)) & 1) << 4));
    }
}

static void unpack_q6k(const uint8_t* b, int8_t* q) { /* values already offset by -32 */
  const uint8_t* ql = b;
  const uint8_t* qh = b + 128;
  for (int h = 0; h < 2; h++)
    for (int l = 0; l < 32; l++) {
      int a = ql[64 * h + l], c = ql[64 * h + 32 + l], hh = qh[32 * h + l];
      q[128 * h + l] = (int8_t)(((a & 0x0F) | (((hh >> 0) & 3) << 4)) - 32);
      q[128 * h + 32 + l] = (int8_t)(((c & 0x0F) | (((hh >> 2) & 3) << 4)) - 32);
      q[128 * h + 64 + l] = (int8_t)(((a >> 4) | (((hh >> 4) & 3) << 4)) - 32);
      q[128 * h + 96 + l] = (int8_t)(((c >> 4) | (((hh >> 6) & 3) << 4)) - 32);
    }
}

/* ------------------------------------------------------------------ dequantize rows
 * Float order (needed for bit-exactness): sub-block scale product first, then times the
 * integer as f32, then the subtraction; every step a separately rounded f32 operation. */

static void dequant_row_q8_0(const uint8_t* b, float* y, int64_t k) {
  for (int64_t ib = 0; ib < k / QK8_0; ib++, b += 34) {
    float d = tqo_f16_to_f32(rd16(b));
    const int8_t* qs = (const int8_t*)(b + 2);
    for (int i = 0; i < QK8_0; i++) y[ib * QK8_0 + i] = (float)qs[i] * d;
  }
}

static void dequant_row_q4k(const uint8_t* b, float* y, int64_t k) {
  int8_t q[QK_K];
  for (int64_t ib = 0; ib < k / QK_K; ib++, b += 144, y += QK_K) {
    float d = tqo_f16_to_f32(rd16(b)), dmin = tqo_f16_to_f32(rd16(b + 2));
    unpack_q4k(b, q);
    for (int j = 0; j < 8; j++) {
      int sc, m;
      k4_scale_min(b + 4, j, &sc, &m);
      float dl = d * (float)sc;
      float ml = dmin * (float)m;
      for (int i = 0; i < 32; i++) {
        float p = dl * (float)q[32 * j + i];
        y[32 * j + i] = p - ml;
      }
    }
  }
}

static void dequant_row_q5k(const uint8_t* b, float* y, int64_t k) {
  int8_t q[QK_K];
  for (int64_t ib = 0; ib < k / QK_K; ib++, b += 176, y += QK_K) {
    float d = tqo_f16_to_f32(rd16(b)), dmin = tqo_f16_to_f32(rd16(b + 2));
    unpack_q5k(b, q);
    for (int j = 0; j < 8; j++) {
      int sc, m;
      k4_scale_min(b + 4, j, &sc, &m);
      float dl = d * (float)sc;
      float ml = dmin * (float)m;
      for (int i = 0; i < 32; i++) {
        float p = dl * (float)q[32 * j + i];
        y[32 * j + i] = p - ml;
      }
    }
  }
}

static void dequant_row_q6k(const uint8_t* b, float* y, int64_t k) {
  int8_t q[QK_K];
  for (int64_t ib = 0; ib < k / QK_K; ib++, b += 210, y += QK_K) {
    float d = tqo_f16_to_f32(rd16(b + 208));
    const int8_t* sc = (const int8_t*)(b + 192);
    unpack_q6k(b, q);
    for (int j = 0; j < 16; j++) {
      float dl = d * (float)sc[j];
      for (int i = 0; i < 16; i++) y[16 * j + i] = dl * (float)q[16 * j + i];
    }
  }
}

static void dequant_row_q8k(const uint8_t* b, float* y, int64_t k) {
  for (int64_t ib = 0; ib < k / QK_K; ib++, b += 292, y += QK_K) {
    float d;
    memcpy(&d, b, 4);
    const int8_t* qs = (const int8_t*)(b + 4);
    for (int i = 0; i < QK_K; i++) y[i] = d * (float)qs[i];
  }
}

static int dequant_row(int dtype, const uint8_t* b, float* y, int64_t k) {
  switch (dtype) {
    case TQO_Q8_0: dequant_row_q8_0(b, y, k); return 0;
    case TQO_Q4_K: dequant_row_q4k(b, y, k); return 0;
    case TQO_Q5_K: dequant_row_q5k(b, y, k); return 0;
    case TQO_Q6_K: dequant_row_q6k(b, y, k); return 0;
    case TQO_Q8_K: dequant_row_q8k(b, y, k); return 0;
    case TQO_F32: memcpy(y, b, (size_t)k * 4); return 0;
    case TQO_F16:
      for (int64_t i = 0; i < k; i++) y[i] = tqo_f16_to_f32(rd16(b + 2 * i));
      return 0;
    case TQO_BF16:
      for (int64_t i = 0; i < k; i++) y[i] = tqo_bf16_to_f32(rd16(b + 2 * i));
      return 0;
    default: return -1;
  }
}

int tqo_dequantize(int dtype, const void* blocks, float* out, int64_t nrows, int64_t k) {
  size_t rb = tqo_row_bytes(dtype, k);
  if (k > 0 && rb == 0) return -1;
  int rc = 0;
#pragma omp parallel for schedule(static) if (nrows > 8)
  for (int64_t r = 0; r < nrows; r++)
    if (dequant_row(dtype, (const uint8_t*)blocks + (size_t)r * rb, out + r * k, k)) rc = -1;
  return rc;
}

/* ------------------------------------------------------------------ quantizers */

/* Q8_0: d = amax/127 kept in f32 for the division, stored as f16; round half away from
 * zero (gguf quants.py:381-393, "bit-exact with the ggml reference"). Used both for
 * weights and, in the CPU matmul scheme, for the activation rows of Q8_0 weights. */
static void quant_row_q8_0(const float* x, uint8_t* b, int64_t k) {
  for (int64_t ib = 0; ib < k / QK8_0; ib++, b += 34, x += QK8_0) {
    float amax = 0.f;
    for (int i = 0; i < QK8_0; i++) {
      float a = fabsf(x[i]);
      if (a > amax) amax = a;
    }
    float d = amax / 127.f;
    float id = d == 0.f ? 0.f : 1.f / d;
    wr16(b, tqo_f32_to_f16(d));
    int8_t* qs = (int8_t*)(b + 2);
    for (int i = 0; i < QK8_0; i++) {
      float v = x[i] * id;
      qs[i] = (int8_t)roundf(v);
    }
  }
}

/* Q8_K activation blocks: f32 d, 256 int8, 16 int16 group sums.
 * Three choices differ between GGML revisions and candle; they are compile-time switches
 * (the CUDA library has the same three under the TURQ_ prefix and must be built alike):
 *   TQO_Q8K_DIVISOR          128 (default) | 127   magnitude the block maximum maps to
 *   TQO_Q8K_NEG_SCALE        1 (default): iscale = -DIVISOR / (signed element of largest
 *                            magnitude, first on ties); 0: iscale = DIVISOR / amax
 *   TQO_Q8K_ROUND_HALF_EVEN  0 (default): ties away from zero, which is what Rust's
 *                            f32::round does and candle-core's BlockQ8K::from_float applies;
 *                            1: ties to even (GGML's nearest_int)
 * The result is clamped at 127 and d = 1/iscale. The defaults restate candle-core's published
 * quantizer; UNPINNED against candle 0.10.2 itself (its source is not in the reference tree). */
#ifndef TQO_Q8K_DIVISOR
#define TQO_Q8K_DIVISOR 128
#endif
#ifndef TQO_Q8K_NEG_SCALE
#define TQO_Q8K_NEG_SCALE 1
#endif
#ifndef TQO_Q8K_ROUND_HALF_EVEN
#define TQO_Q8K_ROUND_HALF_EVEN 0
#endif

int tqo_q8k_variant(void) {
  return TQO_Q8K_DIVISOR | (TQO_Q8K_NEG_SCALE ? 0x100 : 0) | (TQO_Q8K_ROUND_HALF_EVEN ? 0x200 : 0);
}

static void quant_row_q8k(const float* x, uint8_t* b, int64_t k) {
  for (int64_t ib = 0; ib < k / QK_K; ib++, b += 292, x += QK_K) {
    float amax = 0.f, mx = 0.f;
    for (int i = 0; i < QK_K; i++) {
      float a = fabsf(x[i]);
      if (a > amax) {
        amax = a;
        mx = x[i];
      }
    }
    int8_t* qs = (int8_t*)(b + 4);
    int16_t bs[16];
    if (amax == 0.f) {
      memset(b, 0, 292);
      continue;
    }
#if TQO_Q8K_NEG_SCALE
    float iscale = -(float)TQO_Q8K_DIVISOR / mx;
#else
    float iscale = (float)TQO_Q8K_DIVISOR / amax;
#endif
    for (int i = 0; i < QK_K; i++) {
      float v = iscale * x[i];
#if TQO_Q8K_ROUND_HALF_EVEN
      long r = lrintf(v); /* default rounding mode: ties to even */
#else
      long r = (long)roundf(v); /* ties away from zero */
#endif
      qs[i] = (int8_t)(r > 127 ? 127 : r);
    }
    for (int j = 0; j < 16; j++) {
      int s = 0;
      for (int i = 0; i < 16; i++) s += qs[16 * j + i];
      bs[j] = (int16_t)s;
    }
    float d = 1.f / iscale;
    memcpy(b, &d, 4);
    for (int j = 0; j < 16; j++) wr16(b + 260 + 2 * j, (uint16_t)bs[j]);
  }
}

/* Round to nearest, ties to even, with a defined result for every input (lrintf leaves NaN and
 * out-of-range values to the platform): NaN -> 0, otherwise saturating at the int range. Only
 * blocks of non-finite or denormal-range data get there; the device quantizer rounds alike. */
static inline int rint_sat(float v) {
  if (v != v) return 0;
  if (v >= 2147483648.f) return 2147483647;
  if (v <= -2147483648.f) return -2147483647 - 1;
  return (int)lrintf(v);
}

/* Fit x ~ scale*q + mn (mn <= 0) with q in [0,nmax] for one sub-block: min/max start,
 * then alternate rounding and a 2-parameter least-squares refit while the error drops. */
static void fit_scale_min(const float* x, int n, int nmax, float* scale_out, float* negmin_out) {
  float mn = x[0], mx = x[0];
  for (int i = 1; i < n; i++) {
    if (x[i] < mn) mn = x[i];
    if (x[i] > mx) mx = x[i];
  }
  if (mn > 0.f) mn = 0.f;
  if (mx <= mn) {
    *scale_out = 0.f;
    *negmin_out = -mn;
    return;
  }
  float scale = (mx - mn) / (float)nmax;
  float best_err = INFINITY;
  float best_s = scale, best_m = mn;
  for (int it = 0; it < 4; it++) {
    float inv = 1.f / scale;
    double sq = 0, sqq = 0, sx = 0, sxq = 0, err = 0;
    for (int i = 0; i < n; i++) {
      int q = rint_sat((x[i] - mn) * inv);
      q = q < 0 ? 0 : (q > nmax ? nmax : q);
      float r = scale * (float)q + mn - x[i];
      err += (double)r * r;
      sq += q;
      sqq += (double)q * q;
      sx += x[i];
      sxq += (double)x[i] * q;
    }
    if (err < best_err) {
      best_err = (float)err;
      best_s = scale;
      best_m = mn;
    } else {
      break;
    }
    double det = (double)n * sqq - sq * sq;
    if (det <= 0) break;
    double s2 = ((double)n * sxq - sq * sx) / det;
    double m2 = (sx - s2 * sq) / n;
    if (s2 <= 0) break;
    if (m2 > 0) { /* re-solve with the offset pinned at zero */
      m2 = 0;
      s2 = sqq > 0 ? sxq / sqq : s2;
      if (s2 <= 0) break;
    }
    scale = (float)s2;
    mn = (float)m2;
  }
  *scale_out = best_s;
  *negmin_out = -best_m;
}

static void quant_row_q45k(const float* x, uint8_t* b, int64_t k, int bits) {
  const int nmax = (1 << bits) - 1;
  const int bsz = bits == 4 ? 144 : 176;
  for (int64_t ib = 0; ib < k / QK_K; ib++, b += bsz, x += QK_K) {
    float scales[8], mins[8];
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; j++) {
      fit_scale_min(x + 32 * j, 32, nmax, &scales[j], &mins[j]);
      if (scales[j] > max_scale) max_scale = scales[j];
      if (mins[j] > max_min) max_min = mins[j];
    }
    float inv_scale = max_scale > 0.f ? 63.f / max_scale : 0.f;
    float inv_min = max_min > 0.f ? 63.f / max_min : 0.f;
    int ls[8], lm[8];
    for (int j = 0; j < 8; j++) {
      int a = rint_sat(inv_scale * scales[j]);
      int c = rint_sat(inv_min * mins[j]);
      ls[j] = a < 0 ? 0 : (a > 63 ? 63 : a);
      lm[j] = c < 0 ? 0 : (c > 63 ? 63 : c);
    }
    uint16_t dh = tqo_f32_to_f16(max_scale / 63.f), dmh = tqo_f32_to_f16(max_min / 63.f);
    wr16(b, dh);
    wr16(b + 2, dmh);
    k4_pack_scale_min(b + 4, ls, lm);
    float d = tqo_f16_to_f32(dh), dmin = tqo_f16_to_f32(dmh);
    uint8_t L[QK_K];
    for (int j = 0; j < 8; j++) {
      float dl = d * (float)ls[j], ml = dmin * (float)lm[j];
      for (int i = 0; i < 32; i++) {
        int q = 0;
        if (dl != 0.f) {
          q = rint_sat((x[32 * j + i] + ml) / dl);
          q = q < 0 ? 0 : (q > nmax ? nmax : q);
        }
        L[32 * j + i] = (uint8_t)q;
      }
    }
    uint8_t* qh = b + 16;
    uint8_t* qs = b + (bits == 4 ? 16 : 48);
    if (bits == 5) memset(qh, 0, 32);
    for (int g = 0; g < 4; g++)
      for (int i = 0; i < 32; i++) {
        int lo = L[64 * g + i], hi = L[64 * g + 32 + i];
        qs[32 * g + i] = (uint8_t)((lo & 0x0F) | ((hi & 0x0F) << 4));
        if (bits == 5) qh[i] |= (uint8_t)(((lo >> 4) << (2 * g)) | ((hi >> 4) << (2 * g + 1)));
      }
  }
}

static void quant_row_q6k(const float* x, uint8_t* b, int64_t k) {
  for (int64_t ib = 0; ib < k / QK_K; ib++, b += 210, x += QK_K) {
    float scales[16];
    float max_abs_scale = 0.f;
    for (int j = 0; j < 16; j++) {
      const float* xs = x + 16 * j;
      float amax = 0.f, mx = 0.f;
      for (int i = 0; i < 16; i++) {
        float a = fabsf(xs[i]);
        if (a > amax) {
          amax = a;
          mx = xs[i];
        }
      }
      float s = amax == 0.f ? 0.f : mx / -32.f; /* largest magnitude lands on -32 */
      if (s != 0.f) { /* one least-squares refit of the scale on the rounded integers */
        double sxq = 0, sqq = 0;
        for (int i = 0; i < 16; i++) {
          int q = rint_sat(xs[i] / s);
          q = q < -32 ? -32 : (q > 31 ? 31 : q);
          sxq += (double)xs[i] * q;
          sqq += (double)q * q;
        }
        if (sqq > 0 && sxq != 0) s = (float)(sxq / sqq);
      }
      scales[j] = s;
      if (fabsf(s) > max_abs_scale) max_abs_scale = fabsf(s);
    }
    int8_t* sc = (int8_t*)(b + 192);
    if (max_abs_scale == 0.f) {
      memset(b, 0, 210);
      /* q = 0 is stored as 32: low nibble 0, high two bits = 2 */
      memset(b + 128, 0xAA, 64);
      continue;
    }
    uint16_t dh = tqo_f32_to_f16(max_abs_scale / 127.f);
    float d = tqo_f16_to_f32(dh);
    wr16(b + 208, dh);
    uint8_t L[QK_K];
    for (int j = 0; j < 16; j++) {
      int s = d != 0.f ? rint_sat(scales[j] / d) : 0;
      s = s < -128 ? -128 : (s > 127 ? 127 : s);
      sc[j] = (int8_t)s;
      float dl = d * (float)s;
      for (int i = 0; i < 16; i++) {
        int q = 0;
        if (dl != 0.f) {
          q = rint_sat(x[16 * j + i] / dl);
          q = q < -32 ? -32 : (q > 31 ? 31 : q);
        }
        L[16 * j + i] = (uint8_t)(q + 32);
      }
    }
    uint8_t* ql = b;
    uint8_t* qh = b + 128;
    for (int h = 0; h < 2; h++)
      for (int l = 0; l < 32; l++) {
        int q1 = L[128 * h + l], q2 = L[128 * h + 32 + l], q3 = L[128 * h + 64 + l],
            q4 = L[128 * h + 96 + l];
        ql[64 * h + l] = (uint8_t)((q1 & 0x0F) | ((q3 & 0x0F) << 4));
        ql[64 * h + 32 + l] = (uint8_t)((q2 & 0x0F) | ((q4 & 0x0F) << 4));
        qh[32 * h + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
      }
  }
}

static int quant_row(int dtype, const float* x, uint8_t* b, int64_t k) {
  switch (dtype) {
    case TQO_Q8_0: quant_row_q8_0(x, b, k); return 0;
    case TQO_Q4_K: quant_row_q45k(x, b, k, 4); return 0;
    case TQO_Q5_K: quant_row_q45k(x, b, k, 5); return 0;
    case TQO_Q6_K: quant_row_q6k(x, b, k); return 0;
    case TQO_Q8_K: quant_row_q8k(x, b, k); return 0;
    default: return -1;
  }
}

int tqo_quantize(int dtype, const float* x, void* blocks, int64_t nrows, int64_t k) {
  size_t rb = tqo_row_bytes(dtype, k);
  if (rb == 0 && k > 0) return -1;
  if (tqo_block_elems(dtype) <= 1) return -1;
  int rc = 0;
#pragma omp parallel for schedule(static) if (nrows > 8)
  for (int64_t r = 0; r < nrows; r++)
    if (quant_row(dtype, x + r * k, (uint8_t*)blocks + (size_t)r * rb, k)) rc = -1;
  return rc;
}

/* ------------------------------------------------------------------ block dot products
 * CPU scheme of the reference's QMatMul::forward (src/models/layers/linear.rs:24 enters
 * candle-core): integer dot per sub-block, integer sub-block scales, one f32 scale per
 * (super-)block, f32 accumulation across blocks. */

static float dot_q8_0_q8_0(const uint8_t* w, const uint8_t* a, int64_t k) {
  float sumf = 0.f;
  for (int64_t ib = 0; ib < k / QK8_0; ib++, w += 34, a += 34) {
    const int8_t* qw = (const int8_t*)(w + 2);
    const int8_t* qa = (const int8_t*)(a + 2);
    int sumi = 0;
    for (int i = 0; i < QK8_0; i++) sumi += (int)qw[i] * (int)qa[i];
    sumf += (float)sumi * (tqo_f16_to_f32(rd16(w)) * tqo_f16_to_f32(rd16(a)));
  }
  return sumf;
}

static float dot_q45k_q8k(const uint8_t* w, const uint8_t* a, int64_t k, int bits) {
  const int bsz = bits == 4 ? 144 : 176;
  float sumf = 0.f;
  int8_t q[QK_K];
  for (int64_t ib = 0; ib < k / QK_K; ib++, w += bsz, a += 292) {
    float dx;
    memcpy(&dx, a, 4);
    const int8_t* qa = (const int8_t*)(a + 4);
    float d = dx * tqo_f16_to_f32(rd16(w)), dmin = dx * tqo_f16_to_f32(rd16(w + 2));
    if (bits == 4) unpack_q4k(w, q); else unpack_q5k(w, q);
    int sumi = 0, summ = 0;
    for (int j = 0; j < 8; j++) {
      int sc, m;
      k4_scale_min(w + 4, j, &sc, &m);
      int s = 0;
      for (int i = 0; i < 32; i++) s += (int)q[32 * j + i] * (int)qa[32 * j + i];
      sumi += sc * s;
      int bs = (int16_t)rd16(a + 260 + 4 * j) + (int16_t)rd16(a + 260 + 4 * j + 2);
      summ += m * bs;
    }
    sumf += d * (float)sumi - dmin * (float)summ;
  }
  return sumf;
}

static float dot_q6k_q8k(const uint8_t* w, const uint8_t* a, int64_t k) {
  float sumf = 0.f;
  int8_t q[QK_K];
  for (int64_t ib = 0; ib < k / QK_K; ib++, w += 210, a += 292) {
    float dx;
    memcpy(&dx, a, 4);
    const int8_t* qa = (const int8_t*)(a + 4);
    const int8_t* sc = (const int8_t*)(w + 192);
    float d = dx * tqo_f16_to_f32(rd16(w + 208));
    unpack_q6k(w, q);
    int sumi = 0;
    for (int j = 0; j < 16; j++) {
      int s = 0;
      for (int i = 0; i < 16; i++) s += (int)q[16 * j + i] * (int)qa[16 * j + i];
      sumi += (int)sc[j] * s;
    }
    sumf += d * (float)sumi;
  }
  return sumf;
}

float tqo_vec_dot(int dtype, const void* wrow, const void* arow, int64_t k) {
  switch (dtype) {
    case TQO_Q8_0: return dot_q8_0_q8_0((const uint8_t*)wrow, (const uint8_t*)arow, k);
    case TQO_Q4_K: return dot_q45k_q8k((const uint8_t*)wrow, (const uint8_t*)arow, k, 4);
    case TQO_Q5_K: return dot_q45k_q8k((const uint8_t*)wrow, (const uint8_t*)arow, k, 5);
    case TQO_Q6_K: return dot_q6k_q8k((const uint8_t*)wrow, (const uint8_t*)arow, k);
    default: return NAN;
  }
}

int tqo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static int act_type_for(int dtype) {
  switch (dtype) {
    case TQO_Q8_0: return TQO_Q8_0;
    case TQO_Q4_K: case TQO_Q5_K: case TQO_Q6_K: return TQO_Q8_K;
    default: return -1;
  }
}

int tqo_qmatmul(int dtype, const void* w, int64_t n, int64_t k, const float* x, int64_t m,
                float* y, int nthreads) {
  int at = act_type_for(dtype);
  size_t wrb = tqo_row_bytes(dtype, k);
  if (at < 0 || wrb == 0) return -1;
  size_t arb = tqo_row_bytes(at, k);
  uint8_t* act = (uint8_t*)malloc(arb * (size_t)(m > 0 ? m : 1));
  if (!act) return -2;
#ifdef _OPENMP
  int nt = nthreads > 0 ? nthreads : omp_get_max_threads();
#else
  int nt = 1;
  (void)nthreads;
#endif
#pragma omp parallel for schedule(static) num_threads(nt) if (m > 1)
  for (int64_t r = 0; r < m; r++) quant_row(at, x + r * k, act + (size_t)r * arb, k);
#pragma omp parallel for schedule(static) num_threads(nt)
  for (int64_t c = 0; c < n; c++) {
    const uint8_t* wr = (const uint8_t*)w + (size_t)c * wrb;
    for (int64_t r = 0; r < m; r++) y[r * n + c] = tqo_vec_dot(dtype, wr, act + (size_t)r * arb, k);
  }
  free(act);
  return 0;
}

int tqo_matmul_f64(int dtype, const void* w, int64_t n, int64_t k, const float* x, int64_t m,
                   float* y, int nthreads) {
  size_t wrb = tqo_row_bytes(dtype, k);
  if (wrb == 0) return -1;
#ifdef _OPENMP
  int nt = nthreads > 0 ? nthreads : omp_get_max_threads();
#else
  int nt = 1;
  (void)nthreads;
#endif
  int rc = 0;
#pragma omp parallel num_threads(nt)
  {
    float* row = (float*)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t c = 0; c < n; c++) {
      if (!row || dequant_row(dtype, (const uint8_t*)w + (size_t)c * wrb, row, k)) {
        rc = -1;
        continue;
      }
      for (int64_t r = 0; r < m; r++) {
        const float* xr = x + r * k;
        double acc = 0.0;
        for (int64_t i = 0; i < k; i++) acc += (double)xr[i] * (double)row[i];
        y[r * n + c] = (float)acc;
      }
    }
    free(row);
  }
  return rc;
}
