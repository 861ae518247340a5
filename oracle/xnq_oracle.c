/*
 * CPU oracle, scalar part: block formats, unpackers, quantizers, scalar-order dots, matmul driver.
 * TEST INFRASTRUCTURE ONLY (see xnq_oracle.h). Compile with -ffp-contract=off and without -mfma:
 * the reference is Rust, which never contracts a*b+c, so neither may this file.
 *
 * Parity status: Q8_0 pinned by the reference's own known-answer recipes; Q4_0 / Q4_K / Q6_K /
 * Q8_K PARITY UNPINNED (no reference test or fixture exists for them).
 */
#include "xnq_oracle.h"
#include "xnq_oracle_internal.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------
 * binary16 conversion, software, round-to-nearest-even; subnormals and inf/nan handled.
 * Stands in for crate `half` (Cargo.lock: half 2.7.1), whose f16::from_f32 / to_f32 are IEEE.
 * ---------------------------------------------------------------------------------------- */
uint16_t xnqo_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t expo = (x >> 23) & 0xffu;
  uint32_t mant = x & 0x7fffffu;
  if (expo == 0xff) { /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | (mant ? (0x200u | (mant >> 13)) : 0));
  }
  int e = (int)expo - 127 + 15;
  if (e >= 31) return (uint16_t)(sign | 0x7c00u); /* overflow -> inf */
  if (e <= 0) {                                   /* subnormal half or zero */
    if (e < -10) return (uint16_t)sign;
    mant |= 0x800000u;
    const int shift = 14 - e; /* 14..24 */
    uint32_t half_m = mant >> shift;
    const uint32_t rem = mant & ((1u << shift) - 1);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_m & 1))) half_m++;
    return (uint16_t)(sign | half_m);
  }
  uint32_t h = ((uint32_t)e << 10) | (mant >> 13);
  const uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++; /* may carry into the exponent: fine */
  return (uint16_t)(sign | h);
}

float xnqo_f16_to_f32(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t expo = (h >> 10) & 0x1f;
  uint32_t mant = h & 0x3ffu;
  uint32_t out;
  if (expo == 0) {
    if (mant == 0) {
      out = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        mant <<= 1;
        e++;
      } while (!(mant & 0x400u));
      mant &= 0x3ffu;
      out = sign | ((uint32_t)(127 - 15 - e) << 23) | (mant << 13);
    }
  } else if (expo == 31) {
    out = sign | 0x7f800000u | (mant << 13);
  } else {
    out = sign | ((expo + 127 - 15) << 23) | (mant << 13);
  }
  float f;
  memcpy(&f, &out, 4);
  return f;
}

/* ------------------------------------------------------------------------------------------ */
int xnqo_type_size(int dtype) {
  switch (dtype) { /* xn-core/src/quantized/mod.rs:160-179, k_quants.rs:98,134,174,196,205 */
    case XNQO_F32: return 4;
    case XNQO_Q4_0: return (int)sizeof(blk_q4_0);
    case XNQO_Q8_0: return (int)sizeof(blk_q8_0);
    case XNQO_Q4K: return (int)sizeof(blk_q4k);
    case XNQO_Q6K: return (int)sizeof(blk_q6k);
    case XNQO_Q8K: return (int)sizeof(blk_q8k);
  }
  return xnqo_more_type_size(dtype);
}

int xnqo_block_size(int dtype) {
  switch (dtype) { /* mod.rs:182-195 */
    case XNQO_F32: return 1;
    case XNQO_Q4_0:
    case XNQO_Q8_0: return 32;
    case XNQO_Q4K:
    case XNQO_Q6K:
    case XNQO_Q8K: return QK_K;
  }
  return xnqo_more_block_size(dtype);
}

int xnqo_vec_dot_type(int dtype) {
  switch (dtype) { /* k_quants.rs:210,615,1321,1727 */
    case XNQO_Q4_0:
    case XNQO_Q8_0: return XNQO_Q8_0;
    case XNQO_Q4K:
    case XNQO_Q6K:
    case XNQO_Q8K: return XNQO_Q8K;
  }
  return xnqo_more_vec_dot_type(dtype);
}

/* Rust `f32::round`: half away from zero. `as i32` / `as i8` / `as u8` saturate, NaN -> 0. */
static inline int32_t sat_i32(float v) {
  if (v != v) return 0;
  if (v >= 2147483648.0f) return INT32_MAX;
  if (v <= -2147483648.0f) return INT32_MIN;
  return (int32_t)v;
}
static inline int8_t sat_i8(float v) {
  if (v != v) return 0;
  if (v >= 127.0f) return 127;
  if (v <= -128.0f) return -128;
  return (int8_t)v;
}
static inline uint8_t sat_u8(float v) {
  if (v != v) return 0;
  if (v >= 255.0f) return 255;
  if (v <= 0.0f) return 0;
  return (uint8_t)v;
}
/* utils.rs:3-5 */
static inline int32_t nearest_int(float v) { return sat_i32(roundf(v)); }
static inline int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* utils.rs:53-63 */
void xnqo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

/* ==========================================================================================
 * to_float
 * ======================================================================================== */
/* k_quants.rs:213-233 */
static void q4_0_to_float(const blk_q4_0 *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d);
    for (int j = 0; j < 16; j++) {
      const int x0 = (b[i].qs[j] & 0x0F) - 8;
      const int x1 = (b[i].qs[j] >> 4) - 8;
      y[i * 32 + j] = (float)x0 * d;
      y[i * 32 + j + 16] = (float)x1 * d;
    }
  }
}
/* k_quants.rs:618-634 */
static void q8_0_to_float(const blk_q8_0 *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d);
    for (int j = 0; j < 32; j++) y[i * 32 + j] = (float)b[i].qs[j] * d;
  }
}
/* k_quants.rs:1475-1503 */
static void q4k_to_float(const blk_q4k *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d);
    const float mn = xnqo_f16_to_f32(b[i].dmin);
    float *out = y + i * QK_K;
    int is = 0;
    for (int j = 0; j < QK_K; j += 64) {
      const uint8_t *q = b[i].qs + j / 2;
      uint8_t sc, m;
      xnqo_scale_min_k4(is, b[i].scales, &sc, &m);
      const float d1 = d * (float)sc, m1 = mn * (float)m;
      xnqo_scale_min_k4(is + 1, b[i].scales, &sc, &m);
      const float d2 = d * (float)sc, m2 = mn * (float)m;
      for (int l = 0; l < 32; l++) *out++ = d1 * (float)(q[l] & 0xF) - m1;
      for (int l = 0; l < 32; l++) *out++ = d2 * (float)(q[l] >> 4) - m2;
      is += 2;
    }
  }
}
/* k_quants.rs:1874-1904 */
static void q6k_to_float(const blk_q6k *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float d = xnqo_f16_to_f32(b[i].d);
    for (int n = 0; n < QK_K; n += 128) {
      const int idx = n / 128;
      float *ys = y + i * QK_K + n;
      const int8_t *sc = b[i].scales + 8 * idx;
      const uint8_t *ql = b[i].ql + 64 * idx;
      const uint8_t *qh = b[i].qh + 32 * idx;
      for (int l = 0; l < 32; l++) {
        const int is = l / 16;
        const int8_t q1 = (int8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
        const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
        const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
        const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        ys[l] = d * (float)sc[is] * (float)q1; /* left to right: (d*sc)*q */
        ys[l + 32] = d * (float)sc[is + 2] * (float)q2;
        ys[l + 64] = d * (float)sc[is + 4] * (float)q3;
        ys[l + 96] = d * (float)sc[is + 6] * (float)q4;
      }
    }
  }
}
/* k_quants.rs:1981-1992 */
static void q8k_to_float(const blk_q8k *b, int64_t nb, float *y) {
  for (int64_t i = 0; i < nb; i++)
    for (int j = 0; j < QK_K; j++) y[i * QK_K + j] = b[i].d * (float)b[i].qs[j];
}

int xnqo_to_float(int dtype, const void *blocks, int64_t nelem, float *out) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 0 || nelem < 0 || nelem % bs != 0) return -1;
  const int64_t nb = nelem / bs;
  switch (dtype) {
    case XNQO_Q4_0: q4_0_to_float((const blk_q4_0 *)blocks, nb, out); return 0;
    case XNQO_Q8_0: q8_0_to_float((const blk_q8_0 *)blocks, nb, out); return 0;
    case XNQO_Q4K: q4k_to_float((const blk_q4k *)blocks, nb, out); return 0;
    case XNQO_Q6K: q6k_to_float((const blk_q6k *)blocks, nb, out); return 0;
    case XNQO_Q8K: q8k_to_float((const blk_q8k *)blocks, nb, out); return 0;
  }
  return xnqo_more_to_float(dtype, blocks, nb, out);
}

/* ==========================================================================================
 * from_float
 * ======================================================================================== */
/* k_quants.rs:235-270 */
static void q4_0_from_float(const float *x, int64_t nb, blk_q4_0 *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float *xs = x + i * 32;
    float amax = 0.f, max = 0.f;
    for (int j = 0; j < 32; j++) {
      if (amax < fabsf(xs[j])) {
        amax = fabsf(xs[j]);
        max = xs[j];
      }
    }
    const float d = max / -8.0f;
    const float id = d != 0.f ? 1.f / d : 0.f;
    y[i].d = xnqo_f32_to_f16(d);
    for (int j = 0; j < 16; j++) {
      const float x0 = xs[j] * id;
      const float x1 = xs[16 + j] * id;
      uint8_t xi0 = sat_u8(x0 + 8.5f);
      uint8_t xi1 = sat_u8(x1 + 8.5f);
      if (xi0 > 15) xi0 = 15;
      if (xi1 > 15) xi1 = 15;
      y[i].qs[j] = (uint8_t)(xi0 | (xi1 << 4));
    }
  }
}

/* k_quants.rs:636-661. The activation quantizer for Q4_0 / Q8_0 weights. */
void xnqo_q8_0_from_float(const float *x, int64_t nb, blk_q8_0 *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float *xs = x + i * 32;
    float amax = 0.f;
    for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(xs[j])); /* f32::max ignores NaN too */
    const float d = amax / 127.0f;
    const float id = d != 0.f ? 1.f / d : 0.f;
    y[i].d = xnqo_f32_to_f16(d);
    for (int j = 0; j < 32; j++) y[i].qs[j] = sat_i8(roundf(xs[j] * id));
  }
}

/* k_quants.rs:1942-1979. The activation quantizer for Q4_K / Q6_K weights. The reference writes
 * into zero-initialised blocks (k_quants.rs:2019), so an all-zero group leaves bsums at 0. */
void xnqo_q8k_from_float(const float *x, int64_t nb, blk_q8k *y) {
  for (int64_t i = 0; i < nb; i++) {
    const float *xs = x + i * QK_K;
    float max = 0.f, amax = 0.f;
    for (int j = 0; j < QK_K; j++) {
      if (amax < fabsf(xs[j])) {
        amax = fabsf(xs[j]);
        max = xs[j];
      }
    }
    if (amax == 0.f) {
      y[i].d = 0.f;
      memset(y[i].qs, 0, QK_K);
      memset(y[i].bsums, 0, sizeof(y[i].bsums));
      continue;
    }
    const float iscale = -128.f / max;
    for (int j = 0; j < QK_K; j++) {
      const float v = roundf(iscale * xs[j]);
      y[i].qs[j] = sat_i8(fminf(v, 127.f));
    }
    for (int j = 0; j < QK_K / 16; j++) {
      int32_t sum = 0;
      for (int ii = 0; ii < 16; ii++) sum += y[i].qs[j * 16 + ii];
      y[i].bsums[j] = (int16_t)sum;
    }
    y[i].d = 1.0f / iscale;
  }
}

/* utils.rs:205-254 */
static void make_qkx1_quants(int nmax, int ntry, const float *x, int n, float *scale_out, float *min_out) {
  uint8_t l[64];
  memset(l, 0, sizeof(l));
  float min = x[0], max = x[0];
  for (int i = 1; i < n; i++) {
    if (x[i] < min) min = x[i];
    if (x[i] > max) max = x[i];
  }
  if (max == min) {
    *scale_out = 0.f;
    *min_out = 0.f;
    return;
  }
  if (min > 0.f) min = 0.f;
  float iscale = (float)nmax / (max - min);
  float scale = 1.0f / iscale;
  for (int t = 0; t < ntry; t++) {
    float sumlx = 0.f;
    int32_t suml2 = 0;
    int did_change = 0;
    for (int i = 0; i < n; i++) {
      const int32_t li = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
      if ((uint8_t)li != l[i]) {
        l[i] = (uint8_t)li;
        did_change = 1;
      }
      sumlx += (x[i] - min) * (float)li;
      suml2 += li * li;
    }
    scale = sumlx / (float)suml2;
    float sum = 0.f;
    for (int i = 0; i < n; i++) sum += x[i] - scale * (float)l[i];
    min = sum / (float)n;
    if (min > 0.f) min = 0.f;
    iscale = 1.0f / scale;
    if (!did_change) break;
  }
  *scale_out = scale;
  *min_out = -min;
}

/* utils.rs:65-202 */
static float make_qx_quants(int n, int nmax, const float *x, int8_t *ls, int rmse_type) {
  float max = 0.f, amax = 0.f;
  for (int i = 0; i < n; i++) {
    const float ax = fabsf(x[i]);
    if (ax > amax) {
      amax = ax;
      max = x[i];
    }
  }
  if (amax == 0.f) {
    for (int i = 0; i < n; i++) ls[i] = 0;
    return 0.f;
  }
  float iscale = -(float)nmax / max;
  if (rmse_type == 0) {
    for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1));
    return 1.0f / iscale;
  }
  const int weight_type = rmse_type % 2;
  float sumlx = 0.f, suml2 = 0.f;
  for (int i = 0; i < n; i++) {
    const int32_t l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
    ls[i] = (int8_t)(l + nmax);
    const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
    const float lf = (float)l;
    sumlx += w * x[i] * lf;
    suml2 += w * lf * lf;
  }
  float scale = sumlx / suml2;
  float best = scale * sumlx;
  for (int itry = 0; itry < 3; itry++) {
    const float isc = 1.0f / scale;
    float slx = 0.f, sl2 = 0.f;
    int changed = 0;
    for (int i = 0; i < n; i++) {
      const int32_t l = clampi(nearest_int(isc * x[i]), -nmax, nmax - 1);
      if (l + nmax != (int32_t)ls[i]) changed = 1;
      const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
      const float lf = (float)l;
      slx += w * x[i] * lf;
      sl2 += w * lf * lf;
    }
    if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
    for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + clampi(nearest_int(isc * x[i]), -nmax, nmax - 1));
    sumlx = slx;
    suml2 = sl2;
    scale = sumlx / suml2;
    best = scale * sumlx;
  }
  for (int itry = 0; itry < 5; itry++) {
    int n_changed = 0;
    for (int i = 0; i < n; i++) {
      const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
      const int32_t l = (int32_t)ls[i] - nmax;
      float slx = sumlx - w * x[i] * (float)l;
      if (slx > 0.f) {
        float sl2 = suml2 - w * (float)l * (float)l;
        const int32_t new_l = clampi(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
        if (new_l != l) {
          slx += w * x[i] * (float)new_l;
          sl2 += w * (float)new_l * (float)new_l;
          if (sl2 > 0.f && slx * slx * suml2 > sumlx * sumlx * sl2) {
            ls[i] = (int8_t)(nmax + new_l);
            sumlx = slx;
            suml2 = sl2;
            scale = sumlx / suml2;
            best = scale * sumlx;
            n_changed++;
          }
        }
      }
    }
    if (n_changed == 0) break;
  }
  if (rmse_type < 3) return scale;
  for (int is = -4; is < 4; is++) {
    if (is == 0) continue;
    iscale = -((float)nmax + 0.1f * (float)is) / max;
    float slx = 0.f, sl2 = 0.f;
    for (int i = 0; i < n; i++) {
      const int32_t l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
      const float w = weight_type == 1 ? x[i] * x[i] : 1.0f;
      const float lf = (float)l;
      slx += w * x[i] * lf;
      sl2 += w * lf * lf;
    }
    if (sl2 > 0.f && slx * slx > best * sl2) {
      for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1));
      scale = slx / sl2;
      best = scale * slx;
    }
  }
  return scale;
}

/* k_quants.rs:1418-1473 */
static void q4k_from_float(const float *xall, int64_t nb, blk_q4k *y) {
  for (int64_t ib = 0; ib < nb; ib++) {
    const float *x = xall + ib * QK_K;
    blk_q4k *b = &y[ib];
    float mins[8], scales[8];
    for (int j = 0; j < 8; j++) make_qkx1_quants(15, 5, x + 32 * j, 32, &scales[j], &mins[j]);
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; j++) {
      max_scale = fmaxf(scales[j], max_scale);
      max_min = fmaxf(mins[j], max_min);
    }
    const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
    const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
    memset(b->scales, 0, 12);
    for (int j = 0; j < 8; j++) {
      int32_t lsi = nearest_int(inv_scale * scales[j]);
      int32_t lmi = nearest_int(inv_min * mins[j]);
      if (lsi > 63) lsi = 63;
      if (lmi > 63) lmi = 63;
      const uint8_t ls = (uint8_t)lsi, lm = (uint8_t)lmi; /* `as u8` of a value <= 63; negatives do not occur */
      if (j < 4) {
        b->scales[j] = ls;
        b->scales[j + 4] = lm;
      } else {
        b->scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
        b->scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
        b->scales[j] |= (uint8_t)((lm >> 4) << 6);
      }
    }
    b->d = xnqo_f32_to_f16(max_scale / 63.0f);
    b->dmin = xnqo_f32_to_f16(max_min / 63.0f);
    uint8_t l[QK_K];
    memset(l, 0, sizeof(l));
    for (int j = 0; j < 8; j++) {
      uint8_t sc, m;
      xnqo_scale_min_k4(j, b->scales, &sc, &m);
      const float d = xnqo_f16_to_f32(b->d) * (float)sc;
      if (d != 0.f) {
        const float dm = xnqo_f16_to_f32(b->dmin) * (float)m;
        for (int ii = 0; ii < 32; ii++) {
          const int32_t lv = nearest_int((x[32 * j + ii] + dm) / d);
          l[32 * j + ii] = (uint8_t)clampi(lv, 0, 15);
        }
      }
    }
    for (int j = 0; j < QK_K; j += 64)
      for (int lv = 0; lv < 32; lv++) b->qs[(j / 64) * 32 + lv] = (uint8_t)(l[j + lv] | (l[j + lv + 32] << 4));
  }
}

/* k_quants.rs:1801-1871 */
static void q6k_from_float(const float *xall, int64_t nb, blk_q6k *yb) {
  int8_t l[QK_K];
  float scales[QK_K / 16];
  memset(l, 0, sizeof(l));
  for (int64_t ib = 0; ib < nb; ib++) {
    const float *x = xall + ib * QK_K;
    blk_q6k *y = &yb[ib];
    float max_scale = 0.f, max_abs_scale = 0.f;
    for (int g = 0; g < QK_K / 16; g++) {
      const float scale = make_qx_quants(16, 32, x + 16 * g, l + 16 * g, 1);
      scales[g] = scale;
      const float a = fabsf(scale);
      if (a > max_abs_scale) {
        max_abs_scale = a;
        max_scale = scale;
      }
    }
    const float iscale = -128.f / max_scale;
    y->d = xnqo_f32_to_f16(1.0f / iscale);
    for (int g = 0; g < QK_K / 16; g++) {
      int32_t v = nearest_int(iscale * scales[g]);
      if (v > 127) v = 127;
      y->scales[g] = (int8_t)(v < -128 ? -128 : v); /* `as i8` of an i32 wraps in Rust; values here stay >= -128 */
    }
    for (int g = 0; g < QK_K / 16; g++) {
      const float d = xnqo_f16_to_f32(y->d) * (float)y->scales[g];
      if (d == 0.f) continue;
      for (int ii = 0; ii < 16; ii++) {
        const int32_t ll = clampi(nearest_int(x[16 * g + ii] / d), -32, 31);
        l[16 * g + ii] = (int8_t)(ll + 32);
      }
    }
    uint8_t *ql = y->ql, *qh = y->qh;
    for (int j = 0; j < QK_K; j += 128) {
      for (int li = 0; li < 32; li++) {
        const uint8_t q1 = (uint8_t)l[j + li] & 0xF, q2 = (uint8_t)l[j + li + 32] & 0xF;
        const uint8_t q3 = (uint8_t)l[j + li + 64] & 0xF, q4 = (uint8_t)l[j + li + 96] & 0xF;
        ql[li] = (uint8_t)(q1 | (q3 << 4));
        ql[li + 32] = (uint8_t)(q2 | (q4 << 4));
        qh[li] = (uint8_t)((l[j + li] >> 4) | ((l[j + li + 32] >> 4) << 2) | ((l[j + li + 64] >> 4) << 4) |
                           ((l[j + li + 96] >> 4) << 6));
      }
      ql += 64;
      qh += 32;
    }
  }
}

int xnqo_from_float(int dtype, const float *x, int64_t nelem, void *blocks) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 0 || nelem < 0 || nelem % bs != 0) return -1;
  const int64_t nb = nelem / bs;
  switch (dtype) {
    case XNQO_Q4_0: q4_0_from_float(x, nb, (blk_q4_0 *)blocks); return 0;
    case XNQO_Q8_0: xnqo_q8_0_from_float(x, nb, (blk_q8_0 *)blocks); return 0;
    case XNQO_Q4K: q4k_from_float(x, nb, (blk_q4k *)blocks); return 0;
    case XNQO_Q6K: q6k_from_float(x, nb, (blk_q6k *)blocks); return 0;
    case XNQO_Q8K: xnqo_q8k_from_float(x, nb, (blk_q8k *)blocks); return 0;
  }
  return xnqo_more_from_float(dtype, x, nb, blocks);
}

/* ==========================================================================================
 * scalar-order dots (vec_dot_unopt)
 * ======================================================================================== */
/* k_quants.rs:287-304 */
static float dot_q4_0(int64_t nb, const blk_q4_0 *x, const blk_q8_0 *y) {
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    int32_t sumi = 0;
    for (int j = 0; j < 16; j++) {
      const int v0 = (x[i].qs[j] & 0x0F) - 8;
      const int v1 = (x[i].qs[j] >> 4) - 8;
      sumi += v0 * y[i].qs[j] + v1 * y[i].qs[j + 16];
    }
    sumf += (float)sumi * xnqo_f16_to_f32(x[i].d) * xnqo_f16_to_f32(y[i].d);
  }
  return sumf;
}
/* k_quants.rs:677-691 */
static float dot_q8_0(int64_t nb, const blk_q8_0 *x, const blk_q8_0 *y) {
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    int32_t sumi = 0;
    for (int j = 0; j < 32; j++) sumi += (int32_t)x[i].qs[j] * (int32_t)y[i].qs[j];
    sumf += (float)sumi * xnqo_f16_to_f32(x[i].d) * xnqo_f16_to_f32(y[i].d);
  }
  return sumf;
}
/* k_quants.rs:1337-1416 */
static float dot_q4k(int64_t nb, const blk_q4k *xs, const blk_q8k *ys) {
  int8_t aux8[QK_K];
  float sums[8] = {0};
  float sumf = 0.f;
  for (int64_t i = 0; i < nb; i++) {
    const blk_q4k *x = &xs[i];
    const blk_q8k *y = &ys[i];
    int32_t aux32[8] = {0};
    for (int c = 0; c < QK_K / 64; c++) {
      for (int l = 0; l < 32; l++) aux8[64 * c + l] = (int8_t)(x->qs[32 * c + l] & 0xF);
      for (int l = 0; l < 32; l++) aux8[64 * c + 32 + l] = (int8_t)(x->qs[32 * c + l] >> 4);
    }
    uint8_t scales[8], mins[8];
    for (int j = 0; j < 8; j++) xnqo_scale_min_k4(j, x->scales, &scales[j], &mins[j]);
    int32_t sumi = 0;
    for (int j = 0; j < QK_K / 16; j++) sumi += (int32_t)y->bsums[j] * (int32_t)mins[j / 2];
    const int8_t *a = aux8;
    const int8_t *q8 = y->qs;
    for (int s = 0; s < 8; s++) {
      const int32_t scale = scales[s];
      for (int g = 0; g < 4; g++) {
        for (int l = 0; l < 8; l++) aux32[l] += scale * (int32_t)(int16_t)(q8[l] * a[l]);
        q8 += 8;
        a += 8;
      }
    }
    const float d = xnqo_f16_to_f32(x->d) * y->d;
    for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
    const float dmin = xnqo_f16_to_f32(x->dmin) * y->d;
    sumf -= dmin * (float)sumi;
  }
  float tail = 0.f;
  for (int l = 0; l < 8; l++) tail += sums[l];
  return sumf + tail;
}
/* k_quants.rs:1743-1799 */
static float dot_q6k(int64_t nb, const blk_q6k *xs, const blk_q8k *ys) {
  int8_t aux8[QK_K];
  float sums[8] = {0};
  for (int64_t i = 0; i < nb; i++) {
    const blk_q6k *x = &xs[i];
    const blk_q8k *y = &ys[i];
    float aux32[8] = {0};
    for (int j = 0; j < QK_K; j += 128) {
      int8_t *a = aux8 + j;
      const uint8_t *q4 = x->ql + j / 2;
      const uint8_t *qh = x->qh + j / 4;
      for (int l = 0; l < 32; l++) {
        a[l] = (int8_t)((int)((q4[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
        a[l + 32] = (int8_t)((int)((q4[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
        a[l + 64] = (int8_t)((int)((q4[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
        a[l + 96] = (int8_t)((int)((q4[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
      }
    }
    for (int j = 0; j < QK_K / 16; j++) {
      const float scale = (float)x->scales[j];
      const int8_t *q8 = y->qs + 16 * j;
      const int8_t *a = aux8 + 16 * j;
      for (int l = 0; l < 8; l++) aux32[l] += scale * (float)(int16_t)(q8[l] * a[l]);
      for (int l = 0; l < 8; l++) aux32[l] += scale * (float)(int16_t)(q8[8 + l] * a[8 + l]);
    }
    const float d = xnqo_f16_to_f32(x->d) * y->d;
    for (int l = 0; l < 8; l++) sums[l] += aux32[l] * d;
  }
  float tail = 0.f;
  for (int l = 0; l < 8; l++) tail += sums[l];
  return tail;
}

int xnqo_vec_dot(int dtype, int64_t k, const void *w, const void *a, float *out) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 1 || k < 0 || k % bs != 0) return -1;
  const int64_t nb = k / bs;
  switch (dtype) {
    case XNQO_Q4_0: *out = dot_q4_0(nb, (const blk_q4_0 *)w, (const blk_q8_0 *)a); return 0;
    case XNQO_Q8_0: *out = dot_q8_0(nb, (const blk_q8_0 *)w, (const blk_q8_0 *)a); return 0;
    case XNQO_Q4K: *out = dot_q4k(nb, (const blk_q4k *)w, (const blk_q8k *)a); return 0;
    case XNQO_Q6K: *out = dot_q6k(nb, (const blk_q6k *)w, (const blk_q8k *)a); return 0;
  }
  return xnqo_more_vec_dot(dtype, nb, w, a, out);
}

/* ==========================================================================================
 * matmul drivers
 * ======================================================================================== */
/* k_quants.rs:2015-2026: rows quantized one at a time into fresh zeroed blocks */
void *xnqo_quantize_lhs(int dtype, int64_t m, int64_t k, const float *lhs) {
  const int adt = xnqo_vec_dot_type(dtype);
  const int abs_ = xnqo_block_size(adt), ats = xnqo_type_size(adt);
  const int64_t kb = k / abs_;
  void *blocks = calloc((size_t)(m * kb > 0 ? m * kb : 1), (size_t)ats);
  if (!blocks) return NULL;
  for (int64_t r = 0; r < m; r++)
    xnqo_from_float(adt, lhs + r * k, k, (char *)blocks + (size_t)r * kb * ats);
  return blocks;
}

typedef struct {
  int dtype;
  int64_t m, k, n;
  const void *lhs_b;
  const void *rhs;
  float *dst;
  double *dst64;
  const double *lhs_deq; /* f64 path: exact value of every quantized activation */
} mm_job;

static void mm_scalar_worker(int ith, int nth, void *arg) {
  const mm_job *j = (const mm_job *)arg;
  const int wts = xnqo_type_size(j->dtype), wbs = xnqo_block_size(j->dtype);
  const int adt = xnqo_vec_dot_type(j->dtype);
  const int ats = xnqo_type_size(adt), abs_ = xnqo_block_size(adt);
  const size_t wrow = (size_t)(j->k / wbs) * wts, arow = (size_t)(j->k / abs_) * ats;
  const int64_t c0 = j->n * ith / nth, c1 = j->n * (ith + 1) / nth;
  for (int64_t r = 0; r < j->m; r++)
    for (int64_t c = c0; c < c1; c++)
      xnqo_vec_dot(j->dtype, j->k, (const char *)j->rhs + c * wrow, (const char *)j->lhs_b + r * arow,
                   &j->dst[r * j->n + c]);
}

int xnqo_matmul(int dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *rhs, float *dst,
                int threads) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 1 || xnqo_vec_dot_type(dtype) < 0 || dtype == XNQO_Q8K || dtype == XNQO_Q8_1) return -1;
  if (m < 0 || n < 0 || k < 0 || k % bs != 0) return -1;
  /* the dots of Q4_1, Q5_0, Q5_1 refuse an odd number of blocks (k_quants.rs:322-325, 413-415, 523-526) */
  if ((dtype == XNQO_Q4_1 || dtype == XNQO_Q5_0 || dtype == XNQO_Q5_1) && (k / bs) % 2 != 0) return -1;
  if (m == 0 || n == 0) return 0;
  void *lhs_b = xnqo_quantize_lhs(dtype, m, k, lhs);
  if (!lhs_b) return -2;
  mm_job j = {dtype, m, k, n, lhs_b, rhs, dst, NULL, NULL};
  xnqo_pool_run(mm_scalar_worker, &j, threads);
  free(lhs_b);
  return 0;
}

static void mm_f64_worker(int ith, int nth, void *arg) {
  const mm_job *j = (const mm_job *)arg;
  const int wts = xnqo_type_size(j->dtype), wbs = xnqo_block_size(j->dtype);
  const size_t wrow = (size_t)(j->k / wbs) * wts;
  const int64_t c0 = j->n * ith / nth, c1 = j->n * (ith + 1) / nth;
  double *wd = (double *)malloc(sizeof(double) * (size_t)(j->k > 0 ? j->k : 1));
  for (int64_t c = c0; c < c1; c++) {
    const char *wr = (const char *)j->rhs + c * wrow;
    /* exact real value of every weight, in f64 */
    for (int64_t b = 0; b < j->k / wbs; b++) {
      double *o = wd + b * wbs;
      if (j->dtype == XNQO_Q4_0) {
        const blk_q4_0 *x = (const blk_q4_0 *)wr + b;
        const double d = xnqo_f16_to_f32(x->d);
        for (int t = 0; t < 16; t++) {
          o[t] = d * ((x->qs[t] & 0xF) - 8);
          o[t + 16] = d * ((x->qs[t] >> 4) - 8);
        }
      } else if (j->dtype == XNQO_Q8_0) {
        const blk_q8_0 *x = (const blk_q8_0 *)wr + b;
        const double d = xnqo_f16_to_f32(x->d);
        for (int t = 0; t < 32; t++) o[t] = d * x->qs[t];
      } else if (j->dtype == XNQO_Q4K) {
        const blk_q4k *x = (const blk_q4k *)wr + b;
        const double d = xnqo_f16_to_f32(x->d), mn = xnqo_f16_to_f32(x->dmin);
        for (int s = 0; s < 8; s++) {
          uint8_t sc, mm;
          xnqo_scale_min_k4(s, x->scales, &sc, &mm);
          for (int t = 0; t < 32; t++) {
            const uint8_t byte = x->qs[32 * (s / 2) + t];
            const int q = (s & 1) ? (byte >> 4) : (byte & 0xF);
            o[32 * s + t] = d * sc * q - mn * mm;
          }
        }
      } else { /* Q6K */
        const blk_q6k *x = (const blk_q6k *)wr + b;
        const double d = xnqo_f16_to_f32(x->d);
        for (int h = 0; h < 2; h++)
          for (int l = 0; l < 32; l++) {
            const uint8_t *ql = x->ql + 64 * h, *qh = x->qh + 32 * h;
            const int8_t *sc = x->scales + 8 * h;
            const int is = l / 16;
            const int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
            const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            o[128 * h + l] = d * sc[is] * q1;
            o[128 * h + l + 32] = d * sc[is + 2] * q2;
            o[128 * h + l + 64] = d * sc[is + 4] * q3;
            o[128 * h + l + 96] = d * sc[is + 6] * q4;
          }
      }
    }
    for (int64_t r = 0; r < j->m; r++) {
      const double *a = j->lhs_deq + r * j->k;
      double acc = 0.0;
      for (int64_t t = 0; t < j->k; t++) acc += wd[t] * a[t];
      j->dst64[r * j->n + c] = acc;
    }
  }
  free(wd);
}

int xnqo_matmul_f64(int dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *rhs, double *dst,
                    int threads) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 1 || xnqo_vec_dot_type(dtype) < 0 || dtype == XNQO_Q8K || dtype == XNQO_Q8_1) return -1;
  if (m < 0 || n < 0 || k < 0 || k % bs != 0) return -1;
  if (m == 0 || n == 0) return 0;
  void *lhs_b = xnqo_quantize_lhs(dtype, m, k, lhs);
  if (!lhs_b) return -2;
  /* exact value (scale times code, in f64) of every quantized activation */
  double *deq = (double *)malloc(sizeof(double) * (size_t)(m * k > 0 ? m * k : 1));
  if (xnqo_vec_dot_type(dtype) == XNQO_Q8_0) {
    const blk_q8_0 *a = (const blk_q8_0 *)lhs_b;
    for (int64_t b = 0; b < m * k / 32; b++)
      for (int t = 0; t < 32; t++) deq[b * 32 + t] = (double)xnqo_f16_to_f32(a[b].d) * a[b].qs[t];
  } else {
    const blk_q8k *a = (const blk_q8k *)lhs_b;
    for (int64_t b = 0; b < m * k / QK_K; b++)
      for (int t = 0; t < QK_K; t++) deq[b * QK_K + t] = (double)a[b].d * a[b].qs[t];
  }
  mm_job j = {dtype, m, k, n, lhs_b, rhs, NULL, dst, deq};
  xnqo_pool_run(mm_f64_worker, &j, threads);
  free(deq);
  free(lhs_b);
  return 0;
}
