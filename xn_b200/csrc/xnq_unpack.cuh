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

// Device form of a Q4_K header (same 16 bytes as in GGUF): f16 d, f16 dmin, then the sixteen 6-bit
// values re-packed as four 24-bit little-endian fields, one per 64-element group g:
//   field g = sc[2g] | sc[2g+1] << 6 | mn[2g] << 12 | mn[2g+1] << 18
// so a lane that works on group g gets its two scales and two mins with one shift and four masks.
// The GGUF packing (utils.rs:53-63) is restored exactly on read-back.
__device__ __forceinline__ uint32_t k4_field(uint32_t w0, uint32_t w1, uint32_t w2, int g) {
  const uint32_t lo = g < 2 ? w0 : w1, hi = g < 2 ? w1 : w2;
  const int sh = g < 2 ? 24 * g : 24 * g - 32; // 0, 24, 16, 40
  return (uint32_t)((((uint64_t)hi << 32) | lo) >> sh) & 0xffffffu;
}
__device__ __forceinline__ void k4_fields_from_gguf(const uint32_t u[3], uint32_t out[3]) {
  const K4Scales ks = unpack_k4(u[0], u[1], u[2]);
  uint64_t f[4];
#pragma unroll
  for (int g = 0; g < 4; g++) {
    const uint32_t sc0 = k4_byte(ks.sc_lo, ks.sc_hi, 2 * g), sc1 = k4_byte(ks.sc_lo, ks.sc_hi, 2 * g + 1);
    const uint32_t mn0 = k4_byte(ks.mn_lo, ks.mn_hi, 2 * g), mn1 = k4_byte(ks.mn_lo, ks.mn_hi, 2 * g + 1);
    f[g] = sc0 | (sc1 << 6) | (mn0 << 12) | (mn1 << 18);
  }
  out[0] = (uint32_t)(f[0] | (f[1] << 24));
  out[1] = (uint32_t)((f[1] >> 8) | (f[2] << 16));
  out[2] = (uint32_t)((f[2] >> 16) | (f[3] << 8));
}
__device__ __forceinline__ void k4_fields_to_gguf(const uint32_t w[3], uint32_t out[3]) {
  uint32_t sc[8], mn[8];
#pragma unroll
  for (int g = 0; g < 4; g++) {
    const uint32_t f = k4_field(w[0], w[1], w[2], g);
    sc[2 * g] = f & 63;
    sc[2 * g + 1] = (f >> 6) & 63;
    mn[2 * g] = (f >> 12) & 63;
    mn[2 * g + 1] = (f >> 18) & 63;
  }
  out[0] = out[1] = out[2] = 0;
#pragma unroll
  for (int j = 0; j < 4; j++) { // k_quants.rs:1437-1444
    out[0] |= (sc[j] | ((sc[j + 4] >> 4) << 6)) << (8 * j);
    out[1] |= (mn[j] | ((mn[j + 4] >> 4) << 6)) << (8 * j);
    out[2] |= ((sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4)) << (8 * j);
  }
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
  const uint32_t f = k4_field(u[0], u[1], u[2], sub >> 1);
  const float sc = (float)((f >> (6 * (sub & 1))) & 63);
  const float mn = (float)((f >> (12 + 6 * (sub & 1))) & 63);
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
