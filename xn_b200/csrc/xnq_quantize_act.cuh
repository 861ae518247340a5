// Warp-level activation quantization, 8 elements per lane. Shared by the standalone quantizer
// kernel and by matmul kernels that quantize in their prologue, so both produce the same bytes.
//
// Arithmetic follows the reference exactly (IEEE division, round half away from zero, saturating
// int8 cast): BlockQ8_0::from_float k_quants.rs:636-661, BlockQ8K::from_float k_quants.rs:1942-1979.
#pragma once

#include "xnq_common.cuh"

namespace xnq {

struct Quant8 {
  uint32_t lo, hi;   // eight int8 codes, element 0 in the low byte of lo
  float d;           // block scale as the dots use it (Q8_0: f16-rounded then widened; Q8_K: f32)
  float d_unrounded; // Q8_0: the f32 scale before the f16 store
  int sum16;         // sum of the 16 codes of this lane pair (a BlockQ8K::bsums entry)
};

__device__ __forceinline__ void load8(const float *p, float v[8]) {
  const float4 a = *reinterpret_cast<const float4 *>(p);
  const float4 b = *reinterpret_cast<const float4 *>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __half *p, float v[8]) {
  const uint4 raw = *reinterpret_cast<const uint4 *>(p);
  const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float v[8]) {
  const uint4 raw = *reinterpret_cast<const uint4 *>(p);
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// ---- RMSNorm arithmetic, shared by the stand-alone add+RMSNorm kernel and by the one-row matvec that applies the norm in
// its prologue, so that both produce the same bits. The sum of squares of a row has ONE order: each run of 8 consecutive
// elements is summed first (fused multiply-adds, element 0 first), 32 consecutive runs (256 elements) are combined by the
// warp's xor-shuffle tree, and the 256-element partial sums are added in index order.
__device__ __forceinline__ float rms_run_sum(const float (&v)[8]) {
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < 8; e++) s = __fmaf_rn(v[e], v[e], s);
  return s;
}
__device__ __forceinline__ float rms_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float rms_scale(float total, int d, float eps) { return rsqrtf(__fadd_rn(__fdiv_rn(total, (float)d), eps)); }
__device__ __forceinline__ float rms_apply(float v, float r, float g) { return __fmul_rn(__fmul_rn(v, r), g); }

// Rust `f32::round` (half away from zero) followed by `as i8` (saturating, NaN -> 0), for the
// products a quantizer forms (|v| far below 2^22). trunc(v + copysign(0.5, v)) is exact there: v and
// v + 0.5 share a binade whose ulp divides 0.5, or the sum lands just ABOVE a power of two, so the
// addition never rounds up across an integer; the one exception, |v| just under 0.5 (the sum would
// round to 1), is caught by the guard. cvt.rzi of NaN is 0 and of +-inf saturates, as `as` does.
__device__ __forceinline__ int round_away_sat_i8(float v) {
  const int r = __float2int_rz(v + copysignf(0.5f, v));
  return fabsf(v) < 0.5f ? 0 : max(-128, min(127, r));
}

__device__ __forceinline__ void pack8(const int q[8], Quant8 &o) {
  o.lo = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
  o.hi = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
  int s = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  o.sum16 = s;
}

// One Q8_0 block = 4 consecutive lanes. All 32 lanes of the warp must call this.
__device__ __forceinline__ Quant8 quantize8_q8_0(const float v[8], int /*lane*/) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i])); // f32::max: a NaN operand is ignored
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
  int q[8];
#pragma unroll
  for (int i = 0; i < 8; i++) q[i] = round_away_sat_i8(__fmul_rn(v[i], id));
  Quant8 o;
  pack8(q, o);
  o.d_unrounded = d;
  o.d = __half2float(__float2half_rn(d));
  return o;
}

// One Q8_K block = the whole warp (256 elements). `max` is the FIRST element of largest magnitude,
// sign kept (the reference scans with a strict `<`).
__device__ __forceinline__ Quant8 quantize8_q8k(const float v[8], int lane) {
  float amax = 0.f, mx = 0.f;
  int idx = lane * 8;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float a = fabsf(v[i]);
    if (amax < a) {
      amax = a;
      mx = v[i];
      idx = lane * 8 + i;
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
    if (oa > amax || (oa == amax && oi < idx)) {
      amax = oa;
      idx = oi;
    }
  }
  mx = __shfl_sync(0xffffffffu, mx, idx >> 3); // the winning lane's own first-largest element is element idx
  Quant8 o;
  int q[8];
  if (amax == 0.f) {
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = 0;
    pack8(q, o);
    o.d = o.d_unrounded = 0.f;
    return o;
  }
  const float iscale = __fdiv_rn(-128.f, mx);
#pragma unroll
  for (int i = 0; i < 8; i++) q[i] = min(127, round_away_sat_i8(__fmul_rn(iscale, v[i])));
  pack8(q, o);
  o.d = o.d_unrounded = __fdiv_rn(1.0f, iscale);
  return o;
}

} // namespace xnq
