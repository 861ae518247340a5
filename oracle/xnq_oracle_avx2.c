/*
 * CPU oracle, x86 part: the dots in the summation order of the reference's AVX2 kernels, the Q8_0
 * tiled sgemm, and the threaded drivers. This is what xn's CPU path executes on an x86 host
 * (.cargo/config.toml sets target-cpu=native) and therefore the TIMED CPU BASELINE.
 * TEST INFRASTRUCTURE ONLY. Compile with -mavx2 -mfma -mf16c.
 *
 * Only the f32 part of each dot depends on order (the integer sums are exact), so each kernel is
 * described by: which elements land in which of the 8 f32 lanes, one fused multiply-add per block
 * per lane, and the final horizontal sum ((l0+l4)+(l2+l6)) + ((l1+l5)+(l3+l7)).
 */
#include "xnq_oracle.h"
#include "xnq_oracle_internal.h"

#include <immintrin.h>
#include <stdatomic.h>
#include <stdlib.h>
#include <string.h>

int xnqo_have_avx2(void) {
  return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") && __builtin_cpu_supports("f16c");
}

static inline float h2f(uint16_t h) { return _cvtsh_ss(h); }

/* avx.rs:31-39 */
static inline float hsum8(__m256 v) {
  __m128 r = _mm_add_ps(_mm256_extractf128_ps(v, 1), _mm256_castps256_ps128(v));
  r = _mm_add_ps(r, _mm_movehl_ps(r, r));
  r = _mm_add_ss(r, _mm_movehdup_ps(r));
  return _mm_cvtss_f32(r);
}

/* signed i8 x signed i8 -> 8 f32 lanes, lane L = sum of products of elements 4L..4L+3 (avx.rs:13-59) */
static inline __m256 dot_i8_lanes(__m256i x, __m256i y) {
  const __m256i ax = _mm256_sign_epi8(x, x);
  const __m256i sy = _mm256_sign_epi8(y, x);
  const __m256i p16 = _mm256_maddubs_epi16(ax, sy);
  return _mm256_cvtepi32_ps(_mm256_madd_epi16(_mm256_set1_epi16(1), p16));
}

/* avx.rs:62-80 */
static float dot_q4_0_avx2(int64_t nb, const blk_q4_0 *x, const blk_q8_0 *y) {
  __m256 acc = _mm256_setzero_ps();
  const __m256i lowmask = _mm256_set1_epi8(0x0F), eight = _mm256_set1_epi8(8);
  for (int64_t i = 0; i < nb; i++) {
    const __m256 d = _mm256_set1_ps(h2f(x[i].d) * h2f(y[i].d));
    const __m128i packed = _mm_loadu_si128((const __m128i *)x[i].qs);
    __m256i codes = _mm256_set_m128i(_mm_srli_epi16(packed, 4), packed); /* low nibbles | high nibbles */
    codes = _mm256_sub_epi8(_mm256_and_si256(codes, lowmask), eight);
    const __m256i a = _mm256_loadu_si256((const __m256i *)y[i].qs);
    acc = _mm256_fmadd_ps(d, dot_i8_lanes(codes, a), acc);
  }
  return hsum8(acc);
}

/* avx.rs:83-99 */
static float dot_q8_0_avx2(int64_t nb, const blk_q8_0 *x, const blk_q8_0 *y) {
  __m256 acc = _mm256_setzero_ps();
  for (int64_t i = 0; i < nb; i++) {
    const __m256 d = _mm256_set1_ps(h2f(x[i].d) * h2f(y[i].d));
    const __m256i w = _mm256_loadu_si256((const __m256i *)x[i].qs);
    const __m256i a = _mm256_loadu_si256((const __m256i *)y[i].qs);
    acc = _mm256_fmadd_ps(d, dot_i8_lanes(w, a), acc);
  }
  return hsum8(acc);
}

/* avx.rs:662-743 */
static float dot_q4k_avx2(int64_t nb, const blk_q4k *xs, const blk_q8k *ys) {
  const __m256i lowmask = _mm256_set1_epi8(0x0F);
  __m256 acc = _mm256_setzero_ps();
  __m128 acc_m = _mm_setzero_ps();
  for (int64_t i = 0; i < nb; i++) {
    const blk_q4k *x = &xs[i];
    const blk_q8k *y = &ys[i];
    const float d = y->d * h2f(x->d);
    const float dmin = -y->d * h2f(x->dmin);
    uint8_t sc[8], mn[8];
    for (int j = 0; j < 8; j++) xnqo_scale_min_k4(j, x->scales, &sc[j], &mn[j]);
    /* mins: pair sums of bsums, times the sub-block min; 4 lanes, lane i = sub-blocks 2i, 2i+1 */
    const __m256i bs = _mm256_loadu_si256((const __m256i *)y->bsums);
    const __m128i pairs = _mm_hadd_epi16(_mm256_castsi256_si128(bs), _mm256_extracti128_si256(bs, 1));
    const __m128i mins16 = _mm_cvtepu8_epi16(_mm_loadl_epi64((const __m128i *)mn));
    acc_m = _mm_fmadd_ps(_mm_set1_ps(dmin), _mm_cvtepi32_ps(_mm_madd_epi16(mins16, pairs)), acc_m);
    __m256i sumi = _mm256_setzero_si256();
    for (int j = 0; j < QK_K / 64; j++) {
      const __m256i bits = _mm256_loadu_si256((const __m256i *)(x->qs + 32 * j));
      const __m256i lo = _mm256_and_si256(bits, lowmask);
      const __m256i hi = _mm256_and_si256(_mm256_srli_epi16(bits, 4), lowmask);
      const __m256i a_lo = _mm256_loadu_si256((const __m256i *)(y->qs + 64 * j));
      const __m256i a_hi = _mm256_loadu_si256((const __m256i *)(y->qs + 64 * j + 32));
      sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(_mm256_set1_epi16(sc[2 * j]), _mm256_maddubs_epi16(lo, a_lo)));
      sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(_mm256_set1_epi16(sc[2 * j + 1]), _mm256_maddubs_epi16(hi, a_hi)));
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
  }
  acc_m = _mm_add_ps(acc_m, _mm_movehl_ps(acc_m, acc_m));
  acc_m = _mm_add_ss(acc_m, _mm_movehdup_ps(acc_m));
  return hsum8(acc) + _mm_cvtss_f32(acc_m);
}

/* avx.rs:358-443 */
static float dot_q6k_avx2(int64_t nb, const blk_q6k *xs, const blk_q8k *ys) {
  const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3), off = _mm256_set1_epi8(32);
  __m256 acc = _mm256_setzero_ps();
  for (int64_t i = 0; i < nb; i++) {
    const blk_q6k *x = &xs[i];
    const blk_q8k *y = &ys[i];
    const float d = y->d * h2f(x->d);
    __m256i sumi = _mm256_setzero_si256();
    for (int h = 0; h < 2; h++) {
      const __m256i l0 = _mm256_loadu_si256((const __m256i *)(x->ql + 64 * h));
      const __m256i l1 = _mm256_loadu_si256((const __m256i *)(x->ql + 64 * h + 32));
      const __m256i hb = _mm256_loadu_si256((const __m256i *)(x->qh + 32 * h));
      __m256i code[4];
      code[0] = _mm256_or_si256(_mm256_and_si256(l0, m4), _mm256_slli_epi16(_mm256_and_si256(hb, m2), 4));
      code[1] = _mm256_or_si256(_mm256_and_si256(l1, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 2), m2), 4));
      code[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), m4),
                                _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 4), m2), 4));
      code[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), m4),
                                _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 6), m2), 4));
      for (int g = 0; g < 4; g++) {
        const __m256i a = _mm256_loadu_si256((const __m256i *)(y->qs + 128 * h + 32 * g));
        /* (code - 32) * a as pair sums: code*a - 32*a */
        const __m256i p16 = _mm256_sub_epi16(_mm256_maddubs_epi16(code[g], a), _mm256_maddubs_epi16(off, a));
        const int s = 8 * h + 2 * g; /* two 16-element scale groups per 32 elements */
        const __m256i sc16 = _mm256_set_m128i(_mm_set1_epi16(x->scales[s + 1]), _mm_set1_epi16(x->scales[s]));
        sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(sc16, p16));
      }
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
  }
  return hsum8(acc);
}

static float dot_avx2(int dtype, int64_t nb, const void *w, const void *a) {
  switch (dtype) {
    case XNQO_Q4_0: return dot_q4_0_avx2(nb, (const blk_q4_0 *)w, (const blk_q8_0 *)a);
    case XNQO_Q8_0: return dot_q8_0_avx2(nb, (const blk_q8_0 *)w, (const blk_q8_0 *)a);
    case XNQO_Q4K: return dot_q4k_avx2(nb, (const blk_q4k *)w, (const blk_q8k *)a);
    default: return dot_q6k_avx2(nb, (const blk_q6k *)w, (const blk_q8k *)a);
  }
}

int xnqo_vec_dot_avx2(int dtype, int64_t k, const void *w, const void *a, float *out) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 1 || dtype == XNQO_Q8K || xnqo_vec_dot_type(dtype) < 0 || k < 0 || k % bs != 0) return -1;
  if (!xnqo_have_avx2()) return -3;
  *out = dot_avx2(dtype, k / bs, w, a);
  return 0;
}

/* ------------------------------------------------------------------------------------------
 * Q8_0 x Q8_0 tiled sgemm (avx.rs:187-314): register tiles of RM x RN cells, every cell an
 * independent 8-lane accumulator with one fma per k-block, so a cell's value equals the per-cell
 * dot exactly. Tiles are split statically: thread ith takes jobs [duty*ith, duty*(ith+1)).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int64_t k; /* in blocks */
  const blk_q8_0 *a;
  int64_t lda;
  const blk_q8_0 *b;
  int64_t ldb;
  float *c;
  int64_t ldc;
  int ith, nth;
} sgemm_ctx;

static void sgemm_tile(const sgemm_ctx *s, int rm, int rn, int64_t m0, int64_t m, int64_t n0, int64_t n) {
  const int64_t ytiles = (m - m0) / rm, xtiles = (n - n0) / rn, tiles = xtiles * ytiles;
  if (tiles == 0) return;
  const int64_t duty = (tiles + s->nth - 1) / s->nth;
  const int64_t start = duty * s->ith;
  int64_t end = start + duty;
  if (end > tiles) end = tiles;
  for (int64_t job = start; job < end; job++) {
    const int64_t ii = m0 + job / xtiles * rm, jj = n0 + job % xtiles * rn;
    __m256 cv[4][4];
    for (int j = 0; j < rn; j++)
      for (int i = 0; i < rm; i++) cv[j][i] = _mm256_setzero_ps();
    for (int64_t l = 0; l < s->k; l++)
      for (int j = 0; j < rn; j++)
        for (int i = 0; i < rm; i++) {
          const blk_q8_0 *pa = s->a + s->lda * (ii + i) + l;
          const blk_q8_0 *pb = s->b + s->ldb * (jj + j) + l;
          const __m256 lanes = dot_i8_lanes(_mm256_loadu_si256((const __m256i *)pa->qs), _mm256_loadu_si256((const __m256i *)pb->qs));
          cv[j][i] = _mm256_fmadd_ps(_mm256_set1_ps(h2f(pa->d) * h2f(pb->d)), lanes, cv[j][i]);
        }
    for (int j = 0; j < rn; j++)
      for (int i = 0; i < rm; i++) s->c[s->ldc * (jj + j) + (ii + i)] = hsum8(cv[j][i]);
  }
}

/* recursive split into the largest register tile that fits 16 ymm registers (avx.rs:206-266) */
static void sgemm_pack(const sgemm_ctx *s, int64_t m0, int64_t m, int64_t n0, int64_t n) {
  const int mr = (int)((m - m0) < 4 ? (m - m0) : 4), nr = (int)((n - n0) < 4 ? (n - n0) : 4);
  if (mr <= 0 || nr <= 0) return;
  int mc, nc;
  if (mr == 4 && nr >= 2) { mc = 4; nc = 2; }
  else if ((mr == 3 || mr == 2) && nr == 4) { mc = 2; nc = 4; }
  else if (mr == 3 && nr >= 2) { mc = 3; nc = 2; }
  else if (mr == 2 && nr == 3) { mc = 2; nc = 3; }
  else if (mr == 4) { mc = 4; nc = 1; }
  else if (mr == 2 && nr == 2) { mc = 2; nc = 2; }
  else if (mr == 1 && nr == 4) { mc = 1; nc = 4; }
  else if (mr == 3) { mc = 3; nc = 1; }
  else if (mr == 1 && nr == 3) { mc = 1; nc = 3; }
  else if (mr == 2) { mc = 2; nc = 1; }
  else if (nr == 2) { mc = 1; nc = 2; }
  else { mc = 1; nc = 1; }
  sgemm_tile(s, mc, nc, m0, m, n0, n);
  const int64_t mp = m0 + (m - m0) / mc * mc, np = n0 + (n - n0) / nc * nc;
  sgemm_pack(s, mp, m, n0, np);
  sgemm_pack(s, m0, m, np, n);
}

int xnqo_sgemm_q8_0(int64_t m, int64_t n, int64_t kblocks, const void *a, int64_t lda, const void *b, int64_t ldb,
                    float *c, int64_t ldc, int ith, int nth) {
  if (nth <= 0 || ith < 0 || ith >= nth) return -1;
  if (!xnqo_have_avx2()) return -3;
  if (m == 0 || n == 0) return 0;
  sgemm_ctx s = {kblocks, (const blk_q8_0 *)a, lda, (const blk_q8_0 *)b, ldb, c, ldc, ith, nth};
  sgemm_pack(&s, 0, m, 0, n);
  return 0;
}

/* ------------------------------------------------------------------------------------------
 * threaded drivers
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  int dtype;
  int64_t k, n;
  const char *lhs_row;
  const char *rhs;
  size_t wrow;
  float *dst_row;
  atomic_long next_chunk;
} row_job;

/* k_quants.rs:63-84: one activation row; 128-column chunks taken dynamically */
static void by_row_worker(int ith, int nth, void *arg) {
  (void)ith;
  (void)nth;
  row_job *j = (row_job *)arg;
  const int bs = xnqo_block_size(j->dtype);
  const int64_t nchunks = (j->n + 127) / 128;
  for (;;) {
    const long c = atomic_fetch_add_explicit(&j->next_chunk, 1, memory_order_relaxed);
    if (c >= nchunks) break;
    const int64_t c1 = (c + 1) * 128 < j->n ? (c + 1) * 128 : j->n;
    for (int64_t col = c * 128; col < c1; col++)
      j->dst_row[col] = dot_avx2(j->dtype, j->k / bs, j->rhs + col * j->wrow, j->lhs_row);
  }
}

typedef struct {
  int64_t m, n, kb;
  const void *lhs_b;
  const void *rhs;
  float *dst;
} sg_job;

/* k_quants.rs:753-758: roles swapped so the column-major sgemm output lands row-major in dst */
static void sgemm_worker(int ith, int nth, void *arg) {
  const sg_job *j = (const sg_job *)arg;
  xnqo_sgemm_q8_0(j->n, j->m, j->kb, j->rhs, j->kb, j->lhs_b, j->kb, j->dst, j->n, ith, nth);
}

int xnqo_matmul_avx2_prequant(int dtype, int64_t m, int64_t k, int64_t n, const void *lhs_b, const void *rhs,
                              float *dst, int threads) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 1 || dtype == XNQO_Q8K || xnqo_vec_dot_type(dtype) < 0) return -1;
  if (m < 0 || n < 0 || k < 0 || k % bs != 0) return -1;
  if (!xnqo_have_avx2()) return -3;
  if (m == 0 || n == 0) return 0;
  if (threads <= 0) threads = xnqo_hw_threads();
  if (dtype == XNQO_Q8_0) {
    sg_job j = {m, n, k / 32, lhs_b, rhs, dst};
    xnqo_pool_run(sgemm_worker, &j, threads);
    return 0;
  }
  const int adt = xnqo_vec_dot_type(dtype);
  const size_t arow = (size_t)(k / xnqo_block_size(adt)) * xnqo_type_size(adt);
  for (int64_t r = 0; r < m; r++) {
    row_job j;
    j.dtype = dtype;
    j.k = k;
    j.n = n;
    j.lhs_row = (const char *)lhs_b + r * arow;
    j.rhs = (const char *)rhs;
    j.wrow = (size_t)(k / bs) * xnqo_type_size(dtype);
    j.dst_row = dst + r * n;
    atomic_init(&j.next_chunk, 0);
    xnqo_pool_run(by_row_worker, &j, threads);
  }
  return 0;
}

int xnqo_matmul_avx2(int dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *rhs, float *dst,
                     int threads) {
  const int bs = xnqo_block_size(dtype);
  if (bs <= 1 || dtype == XNQO_Q8K || xnqo_vec_dot_type(dtype) < 0) return -1;
  if (m < 0 || n < 0 || k < 0 || k % bs != 0) return -1;
  if (m == 0 || n == 0) return 0;
  void *lhs_b = xnqo_quantize_lhs(dtype, m, k, lhs);
  if (!lhs_b) return -2;
  const int rc = xnqo_matmul_avx2_prequant(dtype, m, k, n, lhs_b, rhs, dst, threads);
  free(lhs_b);
  return rc;
}
