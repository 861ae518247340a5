// Per-format weight producers of the prefill kernel: two threads own one weight row of the tile.
//
// A k-step of a row is handled in two halves that are several k-steps apart in time:
//   issue()  cp.async copies of the row's raw quantized bytes for that k-step into a slot of the
//            thread's PRIVATE shared-memory ring (no other thread reads it, so no barrier is needed:
//            cp.async.wait_group orders the copies before the same thread's loads);
//   store()  read the slot, dequantize to fp16 and write the 8 swizzled 16-byte chunks of the row into
//            the A stage the tensor core reads.
// Keeping DEPTH k-steps of copies in flight per thread hides the HBM latency without holding the bytes
// in registers. Slot sizes are odd multiples of 16 bytes, so a quarter-warp's 128-bit reads of eight
// neighbouring slots fall into eight different bank groups.
//
// Stored k order inside a k-step (the activation image uses the same one, see kpos_* in xnq_prefill.cu):
//   Q8_0, Q6_K  natural
//   Q4_0        chunk 4b + wi = elements [j, j+2, j+16, j+18, j+1, j+3, j+17, j+19] + 32b, j = 4wi
//   Q4_K        chunk wi      = elements [l, l+2, 32+l, 32+l+2, l+1, l+3, 32+l+1, 32+l+3], l = 4wi
#pragma once

#include "xnq_common.cuh"
#include "xnq_unpack.cuh"

namespace xnq {
namespace prefill_rows {

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 0x6400 is 1024.0 in fp16 and its ulp is 1: OR-ing an integer 0..1023 into the low bits gives 1024 + i exactly.
__device__ __forceinline__ __half2 h2_from_bits(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t bits_from_h2(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
// an f16 block scale times the tensor's power-of-two scale (which may itself lie outside the f16 range), as half2
__device__ __forceinline__ __half2 scaled_half2(uint32_t f16_bits, float wscale) {
  return __float2half2_rn(__half2float(__ushort_as_half((unsigned short)f16_bits)) * wscale);
}

// Two threads share a weight row: thread half hf (0/1) produces chunks 4*hf .. 4*hf+3 of the k-step.
// All shared-memory reads of a call are issued before any arithmetic.

struct RowQ4_0 { // half = one 32-element block
  static constexpr int SLOT = 48; // 16 nibble bytes | f16 scale pair | pad   (odd multiple of 16)
  __device__ static __forceinline__ void issue(const WeightView &w, int64_t row, int kt, int hf, uint32_t slot) {
    const int64_t nblk = w.k / QK;
    const int64_t b = min((int64_t)kt * 2 + hf, nblk - 1); // odd block count: the missing block is zeroed in store()
    cp_async16(slot, w.qs + (row * nblk + b) * 16);
    cp_async4(slot + 16, w.d + row * w.dstride + (b & ~(int64_t)1));
  }
  __device__ static __forceinline__ void store(const WeightView &w, uint32_t slot, int kt, int hf, float wscale, uint32_t dst_row, int sw) {
    const uint4 q = lds128(slot);
    const uint32_t dd = lds32(slot + 16);
    const bool ok = (int64_t)kt * 2 + hf < w.k / QK;
    const __half2 d2 = ok ? scaled_half2(hf ? (dd >> 16) : (dd & 0xffffu), wscale) : __float2half2_rn(0.f);
    const __half2 off = h2_from_bits(0x64086408u); // 1032 = 1024 + 8
    const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int wi = 0; wi < 4; wi++) {
      uint32_t o[4];
#pragma unroll
      for (int p = 0; p < 4; p++) { // nibble pairs (p, p+4) of the word
        const __half2 v = h2_from_bits(((wd[wi] >> (4 * p)) & 0x000f000fu) | 0x64006400u);
        o[p] = bits_from_h2(__hmul2(__hsub2(v, off), d2));
      }
      sts128(dst_row + (((hf * 4 + wi) ^ sw) << 4), o[0], o[1], o[2], o[3]);
    }
  }
};

struct RowQ8_0 { // half = one 32-element block
  static constexpr int SLOT = 48; // 32 codes | f16 scale pair | pad
  __device__ static __forceinline__ void issue(const WeightView &w, int64_t row, int kt, int hf, uint32_t slot) {
    const int64_t nblk = w.k / QK;
    const int64_t b = min((int64_t)kt * 2 + hf, nblk - 1);
    const uint8_t *r = w.qs + row * w.k + b * 32;
    cp_async16(slot, r);
    cp_async16(slot + 16, r + 16);
    cp_async4(slot + 32, w.d + row * w.dstride + (b & ~(int64_t)1));
  }
  __device__ static __forceinline__ void store(const WeightView &w, uint32_t slot, int kt, int hf, float wscale, uint32_t dst_row, int sw) {
    const uint4 q[2] = {lds128(slot), lds128(slot + 16)};
    const uint32_t dd = lds32(slot + 32);
    const bool ok = (int64_t)kt * 2 + hf < w.k / QK;
    const __half2 d2 = ok ? scaled_half2(hf ? (dd >> 16) : (dd & 0xffffu), wscale) : __float2half2_rn(0.f);
    const __half2 off = h2_from_bits(0x64806480u); // 1152 = 1024 + 128
#pragma unroll
    for (int c = 0; c < 4; c++) { // chunk = 8 codes
      const uint32_t ww[2] = {((c & 1) ? q[c >> 1].z : q[c >> 1].x) ^ 0x80808080u, ((c & 1) ? q[c >> 1].w : q[c >> 1].y) ^ 0x80808080u};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const __half2 lo = h2_from_bits(__byte_perm(ww[j], 0x64646464u, 0x4140)); // bytes 0,1 -> 1024 + (b + 128)
        const __half2 hi = h2_from_bits(__byte_perm(ww[j], 0x64646464u, 0x4342)); // bytes 2,3
        o[2 * j] = bits_from_h2(__hmul2(__hsub2(lo, off), d2));
        o[2 * j + 1] = bits_from_h2(__hmul2(__hsub2(hi, off), d2));
      }
      sts128(dst_row + (((hf * 4 + c) ^ sw) << 4), o[0], o[1], o[2], o[3]);
    }
  }
};

struct RowQ4K { // half = 16 of the 32 nibble bytes of the k-step's group (words 4*hf .. 4*hf+3)
  static constexpr int SLOT = 48; // header | 16 nibble bytes | pad
  __device__ static __forceinline__ void issue(const WeightView &w, int64_t row, int kt, int hf, uint32_t slot) {
    const int64_t nsb = w.k / QK_K;
    const uint8_t *blk = w.qs + (row * nsb + (kt >> 2)) * 144;
    cp_async16(slot, blk);
    cp_async16(slot + 16, blk + 16 + 32 * (kt & 3) + 16 * hf);
  }
  __device__ static __forceinline__ void store(const WeightView &, uint32_t slot, int kt, int hf, float wscale, uint32_t dst_row, int sw) {
    const int g = kt & 3;
    const uint4 hdr = lds128(slot), q = lds128(slot + 16);
    const __half2 dm = *reinterpret_cast<const __half2 *>(&hdr.x);
    const uint32_t f = k4_field(hdr.y, hdr.z, hdr.w, g);
    const float d = __low2float(dm) * wscale, mn = __high2float(dm) * wscale;
    // value = (d*sc) * code - (dmin*m): low nibbles are sub-block 2g, high nibbles sub-block 2g+1
    const __half2 a_lo = __float2half2_rn(d * (float)(f & 63)), a_hi = __float2half2_rn(d * (float)((f >> 6) & 63));
    const __half2 b_lo = __float2half2_rn(-mn * (float)((f >> 12) & 63)), b_hi = __float2half2_rn(-mn * (float)(f >> 18));
    const __half2 k1024 = h2_from_bits(0x64006400u);
    const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int wi = 0; wi < 4; wi++) {
      uint32_t o[4];
#pragma unroll
      for (int p = 0; p < 4; p++) { // pairs: p=0 (l, l+2) low, p=1 (32+l, 32+l+2) high, p=2 (l+1, l+3) low, p=3 high
        const __half2 c = __hsub2(h2_from_bits(((wd[wi] >> (4 * p)) & 0x000f000fu) | 0x64006400u), k1024);
        o[p] = bits_from_h2((p & 1) ? __hfma2(c, a_hi, b_hi) : __hfma2(c, a_lo, b_lo));
      }
      sts128(dst_row + (((hf * 4 + wi) ^ sw) << 4), o[0], o[1], o[2], o[3]);
    }
  }
};

struct RowQ6K { // half = one 32-element group: hf = 0 takes the nibbles of ql[l], hf = 1 those of ql[l + 32]
  static constexpr int SLOT = 80; // 32 ql bytes | 32 qh bytes | 4 scales | f16 d pair | pad
  __device__ static __forceinline__ void issue(const WeightView &w, int64_t row, int kt, int hf, uint32_t slot) {
    const int64_t nsb = w.k / QK_K;
    const int sb = kt >> 2, s = kt & 3, h = s >> 1, hi_pair = s & 1;
    const int64_t blk = row * nsb + sb;
    cp_async16(slot, w.qs + blk * 128 + 64 * h + 32 * hf);
    cp_async16(slot + 16, w.qs + blk * 128 + 64 * h + 32 * hf + 16);
    cp_async16(slot + 32, w.qh + blk * 64 + 32 * h);
    cp_async16(slot + 48, w.qh + blk * 64 + 32 * h + 16);
    cp_async4(slot + 64, w.sc + blk * 16 + 8 * h + 4 * hi_pair);
    cp_async4(slot + 68, w.d + row * w.dstride + (sb & ~1));
  }
  __device__ static __forceinline__ void store(const WeightView &, uint32_t slot, int kt, int hf, float wscale, uint32_t dst_row, int sw) {
    const int sb = kt >> 2, hi_pair = kt & 1;
    const uint4 ql[2] = {lds128(slot), lds128(slot + 16)};
    const uint4 qh[2] = {lds128(slot + 32), lds128(slot + 48)};
    const uint32_t sc4 = lds32(slot + 64), dd = lds32(slot + 68);
    const float d = __half2float(__ushort_as_half((unsigned short)((sb & 1) ? (dd >> 16) : (dd & 0xffffu)))) * wscale;
    const __half2 off = h2_from_bits(0x64206420u); // 1056 = 1024 + 32
    const int sh = 4 * hi_pair;       // low or high nibble of ql, and which half of qh's four bit pairs
    const int hsh = sh + 2 * hf;      // bit position of this group's two high bits inside a qh byte
#pragma unroll
    for (int c = 0; c < 4; c++) { // chunk of 8 elements l = 8c .. 8c+7
      const uint32_t lw[2] = {(c & 1) ? ql[c >> 1].z : ql[c >> 1].x, (c & 1) ? ql[c >> 1].w : ql[c >> 1].y};
      const uint32_t hw[2] = {(c & 1) ? qh[c >> 1].z : qh[c >> 1].x, (c & 1) ? qh[c >> 1].w : qh[c >> 1].y};
      const int8_t sc = (int8_t)((sc4 >> (8 * (2 * hf + (c >> 1)))) & 0xff);
      const __half2 s2 = __float2half2_rn(d * (float)sc);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const uint32_t code = ((lw[j] >> sh) & 0x0f0f0f0fu) | (((hw[j] >> hsh) << 4) & 0x30303030u);
        const __half2 lo = h2_from_bits(__byte_perm(code, 0x64646464u, 0x4140));
        const __half2 hi = h2_from_bits(__byte_perm(code, 0x64646464u, 0x4342));
        o[2 * j] = bits_from_h2(__hmul2(__hsub2(lo, off), s2));
        o[2 * j + 1] = bits_from_h2(__hmul2(__hsub2(hi, off), s2));
      }
      sts128(dst_row + (((hf * 4 + c) ^ sw) << 4), o[0], o[1], o[2], o[3]);
    }
  }
};

} // namespace prefill_rows
} // namespace xnq
