/* Internal declarations shared by the oracle's translation units. TEST INFRASTRUCTURE ONLY. */
#ifndef XNQ_ORACLE_INTERNAL_H
#define XNQ_ORACLE_INTERNAL_H
#include <stdint.h>

#define QK_K 256

/* Block layouts, xn-core/src/quantized/k_quants.rs:92-205 (all #[repr(C)], no padding). */
#pragma pack(push, 1)
typedef struct { uint16_t d; uint8_t qs[16]; } blk_q4_0;                                   /* 18 */
typedef struct { uint16_t d; int8_t qs[32]; } blk_q8_0;                                    /* 34 */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4k; /* 144 */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } blk_q6k; /* 210 */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8k;                     /* 292 */
typedef struct { uint16_t d; uint16_t m; uint8_t qs[16]; } blk_q4_1;                        /* 20 */
typedef struct { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_0;                     /* 22 */
typedef struct { uint16_t d; uint16_t m; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_1;         /* 24 */
typedef struct { uint16_t d; uint16_t s; int8_t qs[32]; } blk_q8_1;                         /* 36 */
typedef struct { uint8_t scales[16]; uint8_t qs[64]; uint16_t d; uint16_t dmin; } blk_q2k;  /* 84 */
typedef struct { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; } blk_q3k; /* 110 */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; } blk_q5k; /* 176 */
#pragma pack(pop)

_Static_assert(sizeof(blk_q4_1) == 20, "BlockQ4_1");
_Static_assert(sizeof(blk_q5_0) == 22, "BlockQ5_0");
_Static_assert(sizeof(blk_q5_1) == 24, "BlockQ5_1");
_Static_assert(sizeof(blk_q8_1) == 36, "BlockQ8_1");
_Static_assert(sizeof(blk_q2k) == 84, "BlockQ2K");
_Static_assert(sizeof(blk_q3k) == 110, "BlockQ3K");
_Static_assert(sizeof(blk_q5k) == 176, "BlockQ5K");
_Static_assert(sizeof(blk_q4_0) == 18, "BlockQ4_0");
_Static_assert(sizeof(blk_q8_0) == 34, "BlockQ8_0");
_Static_assert(sizeof(blk_q4k) == 144, "BlockQ4K");
_Static_assert(sizeof(blk_q6k) == 210, "BlockQ6K");
_Static_assert(sizeof(blk_q8k) == 292, "BlockQ8K");

void xnqo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn);
void xnqo_q8_0_from_float(const float *x, int64_t nb, blk_q8_0 *y);
void xnqo_q8k_from_float(const float *x, int64_t nb, blk_q8k *y);
void *xnqo_quantize_lhs(int dtype, int64_t m, int64_t k, const float *lhs);

/* The formats beyond Q4_0 / Q8_0 / Q4_K / Q6_K (xnq_oracle_more.c): each returns -1 for a dtype that is not one of theirs. */
int xnqo_more_type_size(int dtype);
int xnqo_more_block_size(int dtype);
int xnqo_more_vec_dot_type(int dtype);
int xnqo_more_to_float(int dtype, const void *blocks, int64_t nb, float *out);
int xnqo_more_from_float(int dtype, const float *x, int64_t nb, void *blocks);
int xnqo_more_vec_dot(int dtype, int64_t nb, const void *w, const void *a, float *out);

/* A persistent worker pool: fn(ith, nth, arg) runs on nth participants (the caller is ith 0).
 * Stands in for xn-core/src/threadpool.rs (spin-then-park workers, dispatch(ith, nth)). */
typedef void (*xnqo_pool_fn)(int ith, int nth, void *arg);
void xnqo_pool_run(xnqo_pool_fn fn, void *arg, int nth);
#endif
