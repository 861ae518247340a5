/*
 * CPU oracle, second part: the GGML formats beyond Q4_0 / Q8_0 / Q4_K / Q6_K.
 *
 * TEST INFRASTRUCTURE ONLY (see xnq_oracle.h). A plain-C restatement of the reference's Rust; every function cites
 * the lines of xn-core/src/quantized/k_quants.rs it follows. PARITY UNPINNED: the reference holds no test, golden vector
 * or fixture for any of these formats.
 *
 * Restated: block layouts, to_float, the scalar-order dots (vec_dot_unopt), the quantizers of Q4_1, Q5_0, Q5_1 and of the
 * activation format Q8_1. Not restated: the search-based weight quantizers of Q2_K, Q3_K and Q5_K (test weights of those
 * formats are random valid blocks) and the AVX2-order dots (these formats are not part of the timed baseline).
 */
#include <math.h>
#include <string.h>

#include "xnq_oracle.h"
#include "xnq_oracle_internal.h"

static inline uint32_t rd_u32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
/* Rust `as u8` / `as i8` of an f32: truncation toward zero, saturating, NaN -> 0 */
static inline uint8_t as_u8(float v) { return v != v ? 0 : (v >= 255.0f ? 255 : (v <= 0.0f ? 0 : (uint8_t)v)); }
static inline int8_t as_i8(float v) { return v != v ? 0 : (v >= 127.0f ? 127 : (v <= -128.0f ? -128 : (int8_t)v)); }
/* Rust f32::min / f32::max: a NaN operand is ignored */
static inline float rmin(float a, float b) { return a != a ? b : (b != b ? a : (a < b ? a : b)); }
static inline float rmax(float a, float b) { return a != a ? b : (b != b ? a : (a > b ? a : b)); }

int xnqo_more_type_size(int dtype) {
  switch (dtype) { /* mod.rs:160-179 */
    case XNQO_Q4_1: return (int)sizeof(blk_q4_1);
    case XNQO_Q5_0: return (int)sizeof(blk_q5_0);
    case XNQO_Q5_1: return (int)sizeof(blk_q5_1);
    case XNQO_Q8_1: return (int)sizeof(blk_q8_1);
    case XNQO_Q2K: return (int)sizeof(blk_q2k);
    case XNQO_Q3K: return (int)sizeof(blk_q3k);
    case XNQO_Q5K: return (int)sizeof(blk_q5k);
  }
  return -1;
}
int xnqo_more_block_size(int dtype) {
  switch (dtype) { /* mod.rs:182-195 */
    case XNQO_Q4_1:
    case XNQO_Q5_0:
    case XNQO_Q5_1:
    case XNQO_Q8_1: return 32;
    case XNQO_Q2K:
    case XNQO_Q3K:
    case XNQO_Q5K: return QK_K;
  }
  return -1;
}
int xnqo_more_vec_dot_type(int dtype) {
  switch (dtype) { /* k_quants.rs:310, 405, 511, 837, 883, 1046, 1510 */
    case XNQO_Q4_1:
    case XNQO_Q5_1:
    case XNQO_Q8_1: return XNQO_Q8_1;
    case XNQO_Q5_0: return XNQO_Q8_0;
    case XNQO_Q2K:
    case XNQO_Q3K:
    case XNQO_Q5K: return XNQO_Q8K;
  }
  return -1;
}

/* ---------------------------------------------------------------------------------------------- to_float */
/* k_quants.rs:379-399 */
static void q4_1_to_float(const blk_q4_1 *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d), m = xnqo_f16_to_f32(b[i].m);
    for (int j = 0; j < 16; j++) {
      y[i * 32 + j] = (float)(b[i].qs[j] & 0x0F) * d + m;
      y[i * 32 + j + 16] = (float)(b[i].qs[j] >> 4) * d + m;
    }
  }
}
/* k_quants.rs:478-502 */
static void q5_0_to_float(const blk_q5_0 *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d);
    const uint32_t qh = rd_u32(b[i].qh);
    for (int j = 0; j < 16; j++) {
      const uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10), xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
      const int32_t x0 = (int32_t)((b[i].qs[j] & 0x0F) | xh0) - 16, x1 = (int32_t)((b[i].qs[j] >> 4) | xh1) - 16;
      y[i * 32 + j] = (float)x0 * d;
      y[i * 32 + j + 16] = (float)x1 * d;
    }
  }
}
/* k_quants.rs:586-612 */
static void q5_1_to_float(const blk_q5_1 *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d), m = xnqo_f16_to_f32(b[i].m);
    const uint32_t qh = rd_u32(b[i].qh);
    for (int j = 0; j < 16; j++) {
      const uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10), xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
      const uint8_t x0 = (uint8_t)((b[i].qs[j] & 0x0F) | xh0), x1 = (uint8_t)((b[i].qs[j] >> 4) | xh1);
      y[i * 32 + j] = (float)x0 * d + m;
      y[i * 32 + j + 16] = (float)x1 * d + m;
    }
  }
}
/* k_quants.rs:1014-1056: per 128 elements four shifts of 32 quant bytes; scale byte = 4-bit scale | 4-bit min << 4 per 16 */
static void q2k_to_float(const blk_q2k *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d), min = xnqo_f16_to_f32(b[i].dmin);
    int is = 0;
    float *yb = y + i * QK_K;
    for (int half = 0; half < 2; half++) {
      const uint8_t *qs = b[i].qs + 32 * half;
      int idx = 0;
      for (int shift = 0; shift < 8; shift += 2) {
        for (int part = 0; part < 2; part++) {
          const uint8_t sc = b[i].scales[is++];
          const float dl = d * (float)(sc & 0xF), ml = min * (float)(sc >> 4);
          for (int l = 0; l < 16; l++) yb[128 * half + idx++] = dl * (float)((qs[16 * part + l] >> shift) & 3) - ml;
        }
      }
    }
  }
}
/* the sixteen 6-bit scales of a Q3_K block as bytes (k_quants.rs:1122-1127, 1268-1274) */
static void q3k_scales(const uint8_t *packed, int8_t out[16]) {
  const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu;
  uint32_t aux[4] = {rd_u32(packed), rd_u32(packed + 4), rd_u32(packed + 8), 0};
  const uint32_t tmp = aux[2];
  aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
  aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
  aux[0] = (aux[0] & kmask2) | (((tmp) & kmask1) << 4);
  aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
  for (int w = 0; w < 4; w++)
    for (int byte = 0; byte < 4; byte++) out[4 * w + byte] = (int8_t)((aux[w] >> (8 * byte)) & 0xff);
}
/* k_quants.rs:1260-1313 */
static void q3k_to_float(const blk_q3k *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    int8_t scales[16];
    q3k_scales(b[i].scales, scales);
    const float d_all = xnqo_f16_to_f32(b[i].d);
    uint8_t m = 1;
    int is = 0;
    float *yb = y + i * QK_K;
    for (int half = 0; half < 2; half++) {
      const uint8_t *qs = b[i].qs + 32 * half;
      for (int sh = 0; sh < 4; sh++) {
        const int shift = 2 * sh;
        for (int part = 0; part < 2; part++) {
          const float dl = d_all * ((float)scales[is] - 32.0f);
          for (int l = 0; l < 16; l++) {
            const int8_t q = (int8_t)((qs[l + 16 * part] >> shift) & 3) - (int8_t)((b[i].hmask[l + 16 * part] & m) == 0 ? 4 : 0);
            yb[128 * half + 32 * sh + 16 * part + l] = dl * (float)q;
          }
          is++;
        }
        m = (uint8_t)(m << 1);
      }
    }
  }
}
/* k_quants.rs:1684-1718 */
static void q5k_to_float(const blk_q5k *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d), min = xnqo_f16_to_f32(b[i].dmin);
    int is = 0;
    uint8_t u1 = 1, u2 = 2;
    float *yb = y + i * QK_K;
    int idx = 0;
    for (int j = 0; j < QK_K; j += 64) {
      const uint8_t *ql = b[i].qs + j / 2;
      uint8_t sc, mn;
      xnqo_scale_min_k4(is, b[i].scales, &sc, &mn);
      const float d1 = d * (float)sc, m1 = min * (float)mn;
      xnqo_scale_min_k4(is + 1, b[i].scales, &sc, &mn);
      const float d2 = d * (float)sc, m2 = min * (float)mn;
      for (int l = 0; l < 32; l++) yb[idx++] = d1 * ((float)(ql[l] & 0xF) + ((b[i].qh[l] & u1) ? 16.f : 0.f)) - m1;
      for (int l = 0; l < 32; l++) yb[idx++] = d2 * ((float)(ql[l] >> 4) + ((b[i].qh[l] & u2) ? 16.f : 0.f)) - m2;
      is += 2;
      u1 = (uint8_t)(u1 << 2);
      u2 = (uint8_t)(u2 << 2);
    }
  }
}

int xnqo_more_to_float(int dtype, const void *blocks, int64_t nb, float *out) {
  switch (dtype) {
    case XNQO_Q4_1: q4_1_to_float((const blk_q4_1 *)blocks, nb, out); return 0;
    case XNQO_Q5_0: q5_0_to_float((const blk_q5_0 *)blocks, nb, out); return 0;
    case XNQO_Q5_1: q5_1_to_float((const blk_q5_1 *)blocks, nb, out); return 0;
    case XNQO_Q2K: q2k_to_float((const blk_q2k *)blocks, nb, out); return 0;
    case XNQO_Q3K: q3k_to_float((const blk_q3k *)blocks, nb, out); return 0;
    case XNQO_Q5K: q5k_to_float((const blk_q5k *)blocks, nb, out); return 0;
  }
  return -1; /* Q8_1: to_float is unimplemented in the reference too (k_quants.rs:875-877) */
}

/* -------------------------------------------------------------------------------------------- from_float */
/* k_quants.rs:345-376 */
static void q4_1_from_float(const float *x, int64_t nb, blk_q4_1 *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float *xs = x + i * 32;
    float min = INFINITY, max = -INFINITY;
    for (int j = 0; j < 32; j++) min = rmin(xs[j], min), max = rmax(xs[j], max);
    const float d = (max - min) / 15.0f, id = d != 0.f ? 1.0f / d : 0.f;
    y[i].d = xnqo_f32_to_f16(d);
    y[i].m = xnqo_f32_to_f16(min);
    for (int j = 0; j < 16; j++) {
      const float x0 = (xs[j] - min) * id, x1 = (xs[16 + j] - min) * id;
      uint8_t xi0 = as_u8(x0 + 0.5f), xi1 = as_u8(x1 + 0.5f);
      if (xi0 > 15) xi0 = 15;
      if (xi1 > 15) xi1 = 15;
      y[i].qs[j] = (uint8_t)(xi0 | (xi1 << 4));
    }
  }
}
/* k_quants.rs:440-475 */
static void q5_0_from_float(const float *x, int64_t nb, blk_q5_0 *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float *xs = x + i * 32;
    float amax = 0.f, max = 0.f;
    for (int j = 0; j < 32; j++)
      if (amax < fabsf(xs[j])) amax = fabsf(xs[j]), max = xs[j];
    const float d = max / -16.0f, id = d != 0.f ? 1.0f / d : 0.f;
    y[i].d = xnqo_f32_to_f16(d);
    uint32_t qh = 0;
    for (int j = 0; j < 16; j++) {
      const float x0 = xs[j] * id, x1 = xs[j + 16] * id;
      int8_t s0 = as_i8(x0 + 16.5f), s1 = as_i8(x1 + 16.5f);
      if (s0 > 31) s0 = 31;
      if (s1 > 31) s1 = 31;
      const uint8_t xi0 = (uint8_t)s0, xi1 = (uint8_t)s1;
      y[i].qs[j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
      qh |= (((uint32_t)xi0 & 0x10u) >> 4) << j;
      qh |= (((uint32_t)xi1 & 0x10u) >> 4) << (j + 16);
    }
    memcpy(y[i].qh, &qh, 4);
  }
}
/* k_quants.rs:547-583 */
static void q5_1_from_float(const float *x, int64_t nb, blk_q5_1 *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float *xs = x + i * 32;
    float min = INFINITY, max = -INFINITY;
    for (int j = 0; j < 32; j++) min = rmin(xs[j], min), max = rmax(xs[j], max);
    const float d = (max - min) / 31.0f, id = d != 0.f ? 1.0f / d : 0.f;
    y[i].d = xnqo_f32_to_f16(d);
    y[i].m = xnqo_f32_to_f16(min);
    uint32_t qh = 0;
    for (int j = 0; j < 16; j++) {
      const float x0 = (xs[j] - min) * id, x1 = (xs[16 + j] - min) * id;
      const uint8_t xi0 = as_u8(x0 + 0.5f), xi1 = as_u8(x1 + 0.5f);
      y[i].qs[j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
      qh |= (((uint32_t)xi0 & 0x10u) >> 4) << j;
      qh |= (((uint32_t)xi1 & 0x10u) >> 4) << (j + 16);
    }
    memcpy(y[i].qh, &qh, 4);
  }
}
/* k_quants.rs:847-873. `ys.s = f16::from_f32(sum as f32) * ys.d` multiplies two f16 values: crate `half` widens both to
 * f32, multiplies and rounds the product back to f16. */
static void q8_1_from_float(const float *x, int64_t nb, blk_q8_1 *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float *xs = x + i * 32;
    float amax = 0.f;
    for (int j = 0; j < 32; j++) amax = rmax(amax, fabsf(xs[j]));
    const float d = amax / 127.0f, id = d != 0.f ? 1.0f / d : 0.f;
    y[i].d = xnqo_f32_to_f16(d);
    int32_t sum = 0;
    for (int j = 0; j < 16; j++) {
      const float v0 = xs[j] * id, v1 = xs[j + 16] * id;
      y[i].qs[j] = as_i8(roundf(v0));
      y[i].qs[j + 16] = as_i8(roundf(v1));
      sum += (int32_t)y[i].qs[j] + (int32_t)y[i].qs[j + 16];
    }
    y[i].s = xnqo_f32_to_f16(xnqo_f16_to_f32(xnqo_f32_to_f16((float)sum)) * xnqo_f16_to_f32(y[i].d));
  }
}

int xnqo_more_from_float(int dtype, const float *x, int64_t nb, void *blocks) {
  switch (dtype) {
    case XNQO_Q4_1: q4_1_from_float(x, nb, (blk_q4_1 *)blocks); return 0;
    case XNQO_Q5_0: q5_0_from_float(x, nb, (blk_q5_0 *)blocks); return 0;
    case XNQO_Q5_1: q5_1_from_float(x, nb, (blk_q5_1 *)blocks); return 0;
    case XNQO_Q8_1: q8_1_from_float(x, nb, (blk_q8_1 *)blocks); return 0;
  }
  return -1;
}

/* --------------------------------------------------------------------------------------- scalar-order dots */
/* k_quants.rs:317-342 */
static float dot_q4_1(int64_t nb, const blk_q4_1 *x, const blk_q8_1 *y) {
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    int32_t sumi = 0;
    for (int j = 0; j < 16; j++) sumi += (int32_t)(x[i].qs[j] & 0x0F) * y[i].qs[j] + (int32_t)(x[i].qs[j] >> 4) * y[i].qs[j + 16];
    sumf += (float)sumi * xnqo_f16_to_f32(x[i].d) * xnqo_f16_to_f32(y[i].d) + xnqo_f16_to_f32(x[i].m) * xnqo_f16_to_f32(y[i].s);
  }
  return sumf;
}
/* k_quants.rs:419-437 */
static float dot_q5_0(int64_t nb, const blk_q5_0 *x, const blk_q8_0 *y) {
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    const uint32_t qh = rd_u32(x[i].qh);
    int32_t sumi = 0;
    for (int j = 0; j < 16; j++) {
      const uint8_t xh0 = (uint8_t)(((qh & (1u << j)) >> j) << 4), xh1 = (uint8_t)((qh & (1u << (j + 16))) >> (j + 12));
      const int32_t x0 = ((int32_t)(x[i].qs[j] & 0x0F) | (int32_t)xh0) - 16, x1 = ((int32_t)(x[i].qs[j] >> 4) | (int32_t)xh1) - 16;
      sumi += x0 * y[i].qs[j] + x1 * y[i].qs[j + 16];
    }
    sumf += (float)sumi * xnqo_f16_to_f32(x[i].d) * xnqo_f16_to_f32(y[i].d);
  }
  return sumf;
}
/* k_quants.rs:518-544 */
static float dot_q5_1(int64_t nb, const blk_q5_1 *x, const blk_q8_1 *y) {
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    const uint32_t qh = rd_u32(x[i].qh);
    int32_t sumi = 0;
    for (int j = 0; j < 16; j++) {
      const uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
      const int32_t x0 = (int32_t)(x[i].qs[j] & 0xF) | (int32_t)xh0, x1 = (int32_t)(x[i].qs[j] >> 4) | (int32_t)xh1;
      sumi += x0 * y[i].qs[j] + x1 * y[i].qs[j + 16];
    }
    sumf += (float)sumi * xnqo_f16_to_f32(x[i].d) * xnqo_f16_to_f32(y[i].d) + xnqo_f16_to_f32(x[i].m) * xnqo_f16_to_f32(y[i].s);
  }
  return sumf;
}
/* k_quants.rs:899-948 */
static float dot_q2k(int64_t nb, const blk_q2k *xs, const blk_q8k *ys) {
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    const blk_q2k *x = &xs[i];
    const blk_q8k *y = &ys[i];
    const uint8_t *q2 = x->qs;
    const int8_t *q8 = y->qs;
    int32_t summs = 0;
    for (int j = 0; j < 16; j++) summs += (int32_t)y->bsums[j] * (int32_t)(x->scales[j] >> 4);
    const float dall = y->d * xnqo_f16_to_f32(x->d), dmin = y->d * xnqo_f16_to_f32(x->dmin);
    int32_t isum = 0;
    int is = 0;
    for (int half = 0; half < 2; half++) {
      for (int shift = 0; shift < 8; shift += 2) {
        int32_t d = x->scales[is++] & 0xF, isuml = 0;
        for (int l = 0; l < 16; l++) isuml += (int32_t)q8[l] * (int32_t)((q2[l] >> shift) & 3);
        isum += d * isuml;
        d = x->scales[is++] & 0xF;
        isuml = 0;
        for (int l = 16; l < 32; l++) isuml += (int32_t)q8[l] * (int32_t)((q2[l] >> shift) & 3);
        isum += d * isuml;
        q8 += 32;
      }
      q2 += 32;
    }
    sumf += dall * (float)isum - dmin * (float)summs;
  }
  return sumf;
}
/* k_quants.rs:1068-1179 */
static float dot_q3k(int64_t nb, const blk_q3k *xs, const blk_q8k *ys) {
  int8_t aux8[QK_K];
  float sums[8] = {0};
  for (int64_t i = 0; i < nb; i++) {
    const blk_q3k *x = &xs[i];
    const blk_q8k *y = &ys[i];
    const uint8_t *q3 = x->qs;
    int32_t aux32[8] = {0};
    int8_t *a = aux8;
    uint8_t m = 1;
    for (int half = 0; half < 2; half++) {
      for (int shift = 0; shift < 8; shift += 2) {
        for (int l = 0; l < 32; l++) a[l] = (int8_t)((q3[l] >> shift) & 3) - (int8_t)((x->hmask[l] & m) ? 0 : 4);
        a += 32;
        m = (uint8_t)(m << 1);
      }
      q3 += 32;
    }
    int8_t scales[16];
    q3k_scales(x->scales, scales);
    const int8_t *q8 = y->qs;
    a = aux8;
    for (int s = 0; s < 16; s++) {
      const int32_t scale = (int32_t)scales[s] - 32;
      for (int rep = 0; rep < 2; rep++) {
        for (int l = 0; l < 8; l++) aux32[l] += scale * (int32_t)(int16_t)((int16_t)q8[l] * (int16_t)a[l]);
        q8 += 8;
        a += 8;
      }
    }
    const float d = xnqo_f16_to_f32(x->d) * y->d;
    for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
  }
  float tot = 0.f;
  for (int l = 0; l < 8; l++) tot += sums[l];
  return tot;
}
/* k_quants.rs:1523-1607 */
static float dot_q5k(int64_t nb, const blk_q5k *xs, const blk_q8k *ys) {
  const uint32_t kmask1 = 0x3f3f3f3fu, kmask2 = 0x0f0f0f0fu, kmask3 = 0x03030303u;
  int8_t aux8[QK_K];
  float sums[8] = {0};
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    const blk_q5k *x = &xs[i];
    const blk_q8k *y = &ys[i];
    const uint8_t *q5 = x->qs, *hm = x->qh;
    int32_t aux32[8] = {0};
    int8_t *a = aux8;
    uint8_t m = 1;
    for (int c = 0; c < QK_K / 64; c++) {
      for (int l = 0; l < 32; l++) a[l] = (int8_t)((q5[l] & 0xF) + ((hm[l] & m) ? 16 : 0));
      a += 32;
      m = (uint8_t)(m << 1);
      for (int l = 0; l < 32; l++) a[l] = (int8_t)((q5[l] >> 4) + ((hm[l] & m) ? 16 : 0));
      a += 32;
      m = (uint8_t)(m << 1);
      q5 += 32;
    }
    uint32_t utmp[4] = {rd_u32(x->scales), rd_u32(x->scales + 4), rd_u32(x->scales + 8), 0};
    utmp[3] = ((utmp[2] >> 4) & kmask2) | (((utmp[1] >> 6) & kmask3) << 4);
    const uint32_t uaux = utmp[1] & kmask1;
    utmp[1] = (utmp[2] & kmask2) | (((utmp[0] >> 6) & kmask3) << 4);
    utmp[2] = uaux;
    utmp[0] &= kmask1;
    uint8_t scales[8], mins[8];
    for (int w = 0; w < 2; w++)
      for (int byte = 0; byte < 4; byte++) {
        scales[4 * w + byte] = (uint8_t)((utmp[w] >> (8 * byte)) & 0xff);
        mins[4 * w + byte] = (uint8_t)((utmp[2 + w] >> (8 * byte)) & 0xff);
      }
    int32_t sumi = 0;
    for (int j = 0; j < QK_K / 16; j++) sumi += (int32_t)y->bsums[j] * (int32_t)mins[j / 2];
    const int8_t *q8 = y->qs;
    a = aux8;
    for (int s = 0; s < 8; s++) {
      const int32_t scale = scales[s];
      for (int rep = 0; rep < 4; rep++) {
        for (int l = 0; l < 8; l++) aux32[l] += scale * (int32_t)(int16_t)((int16_t)q8[l] * (int16_t)a[l]);
        q8 += 8;
        a += 8;
      }
    }
    const float d = xnqo_f16_to_f32(x->d) * y->d;
    for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
    const float dmin = xnqo_f16_to_f32(x->dmin) * y->d;
    sumf -= dmin * (float)sumi;
  }
  float tot = 0.f;
  for (int l = 0; l < 8; l++) tot += sums[l];
  return sumf + tot;
}

int xnqo_more_vec_dot(int dtype, int64_t nb, const void *w, const void *a, float *out) {
  switch (dtype) {
    /* the 32-element formats refuse an odd number of blocks (k_quants.rs:322-325, 413-415, 523-526) */
    case XNQO_Q4_1: if (nb % 2) return -1; *out = dot_q4_1(nb, (const blk_q4_1 *)w, (const blk_q8_1 *)a); return 0;
    case XNQO_Q5_0: if (nb % 2) return -1; *out = dot_q5_0(nb, (const blk_q5_0 *)w, (const blk_q8_0 *)a); return 0;
    case XNQO_Q5_1: if (nb % 2) return -1; *out = dot_q5_1(nb, (const blk_q5_1 *)w, (const blk_q8_1 *)a); return 0;
    case XNQO_Q2K: *out = dot_q2k(nb, (const blk_q2k *)w, (const blk_q8k *)a); return 0;
    case XNQO_Q3K: *out = dot_q3k(nb, (const blk_q3k *)w, (const blk_q8k *)a); return 0;
    case XNQO_Q5K: *out = dot_q5k(nb, (const blk_q5k *)w, (const blk_q8k *)a); return 0;
  }
  return -1;
}
