// Block unpacking shared by the dequantize, matvec and prefill kernels.
//
// The per-element functions follow GgmlType::to_float operation for operation
// (xn-core/src/quantized/k_quants.rs:213-233, 618-634, 1475-1503, 1874-1904) with explicit
// round-to-nearest intrinsics, so the compiler cannot fuse a multiply and a subtract into one FMA
// and change the last bit.
#pragma once

#include "xnq_common.cuh"

namespace xnq {

// The 12 scale bytes of a Q4_K super-block as three little-endian words -> eight 6-bit scales
// (sc_lo = sub-blocks 0..3, sc_hi = 4..7, one per byte) and eight 6-bit mins, the word-parallel
// form of get_scale_min_k4 (xn-core/src/quantized/utils.rs:53-63).
struct K4Scales {
  uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
};
__device__ __forceinline__ K4Scales unpack_k4(uint32_t u0, uint32_t u1, uint32_t u2) {
  K4Scales r;
  r.sc_lo = u0 & 0x3f3f3f3fu;
  r.mn_lo = u1 & 0x3f3f3f3fu;
  r.sc_hi = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
  r.mn_hi = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
  return r;
}
__device__ __forceinline__ uint32_t k4_byte(uint32_t lo, uint32_t hi, int j) { // j in 0..7
  return ((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xffu;
}

__device__ __forceinline__ float deq_q4_0(const WeightView &w, int64_t row, int col) {
  const int64_t nblk = w.k / QK;
  const int b = col / QK, j = col % QK;
  const uint8_t byte = w.qs[(row * nblk + b) * 16 + (j & 15)];
  const int code = (j < 16 ? (byte & 0xF) : (byte >> 4)) - 8;
  return __fmul_rn((float)code, __half2float(w.d[row * w.dstride + b]));
}

__device__ __forceinline__ float deq_q8_0(const WeightView &w, int64_t row, int col) {
  const int8_t q = reinterpret_cast<const int8_t *>(w.qs)[row * w.k + col];
  return __fmul_rn((float)q, __half2float(w.d[row * w.dstride + col / QK]));
}

__device__ __forceinline__ float deq_q4k(const WeightView &w, int64_t row, int col) {
  const int64_t nsb = w.k / QK_K;
  const uint8_t *blk = w.qs + (row * nsb + col / QK_K) * 144;
  const int e = col % QK_K, sub = e / 32, l = e % 32;
  const __half2 dm = *reinterpret_cast<const __half2 *>(blk);
  const uint32_t *u = reinterpret_cast<const uint32_t *>(blk + 4);
  const K4Scales ks = unpack_k4(u[0], u[1], u[2]);
  const float sc = (float)k4_byte(ks.sc_lo, ks.sc_hi, sub);
  const float mn = (float)k4_byte(ks.mn_lo, ks.mn_hi, sub);
  const uint8_t byte = blk[16 + 32 * (sub >> 1) + l];
  const float code = (float)((sub & 1) ? (byte >> 4) : (byte & 0xF));
  const float d1 = __fmul_rn(__low2float(dm), sc);
  const float m1 = __fmul_rn(__high2float(dm), mn);
  return __fsub_rn(__fmul_rn(d1, code), m1);
}

__device__ __forceinline__ float deq_q6k(const WeightView &w, int64_t row, int col) {
  const int64_t nsb = w.k / QK_K;
  const int64_t blk = row * nsb + col / QK_K;
  const int e = col % QK_K, h = e / 128, r = e % 128, g = r / 32, l = r % 32;
  const uint8_t lb = w.qs[blk * 128 + 64 * h + l + 32 * (g & 1)];
  const int low4 = g >= 2 ? (lb >> 4) : (lb & 0xF);
  const int high2 = (w.qh[blk * 64 + 32 * h + l] >> (2 * g)) & 3;
  const int code = (low4 | (high2 << 4)) - 32;
  const float sc = (float)w.sc[blk * 16 + 8 * h + l / 16 + 2 * g];
  const float d = __half2float(w.d[row * w.dstride + col / QK_K]);
  return __fmul_rn(__fmul_rn(d, sc), (float)code);
}

} // namespace xnq
