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
#pragma pack(pop)

_Static_assert(sizeof(blk_q4_0) == 18, "BlockQ4_0");
_Static_assert(sizeof(blk_q8_0) == 34, "BlockQ8_0");
_Static_assert(sizeof(blk_q4k) == 144, "BlockQ4K");
_Static_assert(sizeof(blk_q6k) == 210, "BlockQ6K");
_Static_assert(sizeof(blk_q8k) == 292, "BlockQ8K");

void xnqo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn);
void xnqo_q8_0_from_float(const float *x, int64_t nb, blk_q8_0 *y);
void xnqo_q8k_from_float(const float *x, int64_t nb, blk_q8k *y);
void *xnqo_quantize_lhs(int dtype, int64_t m, int64_t k, const float *lhs);

/* A persistent worker pool: fn(ith, nth, arg) runs on nth participants (the caller is ith 0).
 * Stands in for xn-core/src/threadpool.rs (spin-then-park workers, dispatch(ith, nth)). */
typedef void (*xnqo_pool_fn)(int ith, int nth, void *arg);
void xnqo_pool_run(xnqo_pool_fn fn, void *arg, int nth);
#endif
