/*
 * CPU oracle for the GGUF block-quantized matmul path of xn-core.
 *
 * TEST INFRASTRUCTURE ONLY. This library is the checker the parity tests compare the CUDA path
 * against, and the timed CPU baseline of the benchmark. Nothing in the shipped library links,
 * loads or calls it.
 *
 * It is a plain-C restatement of the reference's Rust (the Rust original cannot be built where
 * this library is developed: no cargo/rustc). Every function cites the reference file:line it
 * follows (paths relative to the xn repository root).
 *
 * Pinning status. Q8_0 is pinned by re-running the reference's own known-answer recipes
 * (closed-form inputs, f64 dot of the quantized operands, 1e-4: xn-core/src/quantized/k_quants.rs:2155-2210;
 * "tiled sgemm == per-cell vec_dot exactly": xn-core/tests/quantized_tests.rs:125-218), and its
 * block layout and to_float by the output of the reference's own CUDA kernel dequant_q8_f32
 * (xn-core/cuda-kernels/reduce.cu, compiled unmodified by `make ref`), bit for bit.
 * Q4_0, Q4_K, Q6_K and the Q8_K activation quantizer: PARITY UNPINNED - the reference holds no
 * test, golden vector or fixture for them, so this restatement is checked only against the source
 * text of k_quants.rs (struct sizes, round trips, scalar-vs-AVX2 agreement, f64 dots).
 * Q4_1, Q5_0, Q5_1, Q8_1, Q2_K, Q3_K, Q5_K (xnq_oracle_more.c): PARITY UNPINNED for the same reason; to_float,
 * the scalar-order dots and the simple quantizers are restated, the search-based weight quantizers of the K formats
 * and the AVX2-order dots are not (their test weights are synthesized as random valid blocks).
 */
#ifndef XNQ_ORACLE_H
#define XNQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML dtype ids, xn-core/src/quantized/mod.rs:97-137 */
enum {
  XNQO_F32 = 0,
  XNQO_Q4_0 = 2,
  XNQO_Q4_1 = 3,
  XNQO_Q5_0 = 6,
  XNQO_Q5_1 = 7,
  XNQO_Q8_0 = 8,
  XNQO_Q8_1 = 9,
  XNQO_Q2K = 10,
  XNQO_Q3K = 11,
  XNQO_Q4K = 12,
  XNQO_Q5K = 13,
  XNQO_Q6K = 14,
  XNQO_Q8K = 15,
};

/* bytes per block / elements per block (mod.rs:160-195); -1 for an unsupported dtype */
int xnqo_type_size(int dtype);
int xnqo_block_size(int dtype);
/* the activation block format a weight format is dotted against (GgmlType::VecDotType) */
int xnqo_vec_dot_type(int dtype);

/* IEEE binary16 <-> binary32, round-to-nearest-even (crate `half` 2.7.1 semantics) */
uint16_t xnqo_f32_to_f16(float f);
float xnqo_f16_to_f32(uint16_t h);

/* GgmlType::to_float: blocks -> nelem floats. Returns 0, or -1 on a bad dtype / size. */
int xnqo_to_float(int dtype, const void *blocks, int64_t nelem, float *out);
/* GgmlType::from_float: nelem floats -> blocks (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q4K, Q6K, Q8K). */
int xnqo_from_float(int dtype, const float *x, int64_t nelem, void *blocks);

/* GgmlType::vec_dot_unopt (scalar summation order): one k-deep dot of a weight row with the
 * activation row quantized to the weight format's VecDotType. */
int xnqo_vec_dot(int dtype, int64_t k, const void *w_row, const void *act_row, float *out);
/* The same dot in the summation order of the reference's AVX2 kernels (what its x86 build runs). */
int xnqo_vec_dot_avx2(int dtype, int64_t k, const void *w_row, const void *act_row, float *out);

/* k_quants::matmul (k_quants.rs:1997-2011): quantize lhs rows, then every (row, col) cell by the
 * scalar-order dot. `threads` only splits columns; each cell is computed by one thread, so the
 * result does not depend on it. dst is [m, n] row-major. */
int xnqo_matmul(int dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *rhs,
                float *dst, int threads);
/* f64 dot of the *quantized* operands (the reference's own test oracle, k_quants.rs:2162-2184,
 * extended to the other formats by dequantizing both sides exactly in f64). */
int xnqo_matmul_f64(int dtype, int64_t m, int64_t k, int64_t n, const float *lhs,
                    const void *rhs, double *dst, int threads);
/* The reference's x86 execution: AVX2-order dots driven as matmul_by_row (rows serial, 128-column
 * chunks handed out dynamically, k_quants.rs:53-90) or, for Q8_0, the tiled sgemm with a static
 * tile split per thread (k_quants.rs:721-760, avx.rs:199-314). This is the timed CPU baseline. */
int xnqo_matmul_avx2(int dtype, int64_t m, int64_t k, int64_t n, const float *lhs,
                     const void *rhs, float *dst, int threads);
/* Only the second half of xnqo_matmul_avx2 (lhs already quantized), so a benchmark can time
 * quantization and dots separately. */
int xnqo_matmul_avx2_prequant(int dtype, int64_t m, int64_t k, int64_t n, const void *lhs_blocks,
                              const void *rhs, float *dst, int threads);
/* Q8_0 x Q8_0 tiled sgemm alone (avx.rs:115-314): column-major c[ldc*j+i], a is [m,k], b is [n,k]
 * in blocks; ith/nth as in the reference. */
int xnqo_sgemm_q8_0(int64_t m, int64_t n, int64_t kblocks, const void *a, int64_t lda,
                    const void *b, int64_t ldb, float *c, int64_t ldc, int ith, int nth);

/* 1 when the AVX2 paths were compiled in and the CPU running this supports them */
int xnqo_have_avx2(void);
int xnqo_hw_threads(void);

#ifdef __cplusplus
}
#endif
#endif
