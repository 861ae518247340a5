// Decode kernels (m <= 16): dequant-fused quantized matvec, HBM-bound.
//
//   y[r, n] = sum over blocks of  d_w * d_a * (integer dot of codes)          (+ min / offset terms)
//
// which is the arithmetic of the reference's CPU dots (xn-core/src/quantized/k_quants.rs:287-304
// Q4_0, 677-691 Q8_0, 1337-1416 Q4_K, 1743-1799 Q6_K): exact integer sums per (sub-)block, scales
// applied in f32, f32 accumulation. Only the f32 summation order differs (lanes, then a shuffle
// tree), as it already does between the reference's scalar and AVX2 builds.
//
// Mapping. A warp owns R consecutive weight rows and walks k; every lane loads one 16-byte chunk
// of each row per step with a streaming (no-L1-allocate) 128-bit load, unpacks the 4/6/8-bit codes
// in registers, and runs dp4a against the int8 activations, which the CTA staged in shared memory
// once. Activation registers are reused across the R rows, shared-memory traffic per weight byte
// drops by R. Partial sums are reduced with warp shuffles; lane 0 stores.
#include <algorithm>

#include "xnq_common.cuh"
#include "xnq_unpack.cuh"

namespace xnq {

namespace {

int g_sms = 148; // set by matvec_init
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ int dot16(const uint4 &w, const int4 &a, int acc) {
  acc = __dp4a((int)w.x, a.x, acc);
  acc = __dp4a((int)w.y, a.y, acc);
  acc = __dp4a((int)w.z, a.z, acc);
  acc = __dp4a((int)w.w, a.w, acc);
  return acc;
}
__device__ __forceinline__ uint4 and4(const uint4 &v, uint32_t m) { return make_uint4(v.x & m, v.y & m, v.z & m, v.w & m); }
__device__ __forceinline__ uint4 shr4(const uint4 &v, int s) { return make_uint4(v.x >> s, v.y >> s, v.z >> s, v.w >> s); }
__device__ __forceinline__ uint4 shl4(const uint4 &v, int s) { return make_uint4(v.x << s, v.y << s, v.z << s, v.w << s); }
__device__ __forceinline__ uint4 or4(const uint4 &a, const uint4 &b) { return make_uint4(a.x | b.x, a.y | b.y, a.z | b.z, a.w | b.w); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

__device__ __forceinline__ void store_y(void *y, int y_dtype, int64_t idx, float v) {
  if (y_dtype == XNQ_F32) {
    static_cast<float *>(y)[idx] = v;
  } else if (y_dtype == XNQ_F16) {
    static_cast<__half *>(y)[idx] = __float2half_rn(v);
  } else {
    static_cast<__nv_bfloat16 *>(y)[idx] = __float2bfloat16_rn(v);
  }
}

// Shared-memory image of the quantized activations: q [m][k] int8 | d [m][nblk] f32 | bsum [m][k/16] i16
struct SmemAct {
  const int8_t *q;
  const float *d;
  const int16_t *bsum;
};
__host__ __device__ inline size_t smem_act_bytes(int64_t m, int64_t k, int blk, bool with_bsum) {
  size_t b = (size_t)m * k;                                  // multiple of 32
  b += (((size_t)m * (k / blk) * 4) + 15) & ~(size_t)15;
  if (with_bsum) b += (((size_t)m * (k / 16) * 2) + 15) & ~(size_t)15;
  return b;
}

// swizzle: 16-byte chunk g of the codes sits at chunk g ^ (((g >> 3) & 3) << 1). A 128-bit shared load is served a
// quarter warp at a time; the eight lanes of a quarter read chunks that differ in bits 0, 3 and 4 of g only (16-element
// half, half of the 256-element block, odd / even block), so without the swizzle they fall into two of the eight bank
// groups (four wavefronts per quarter) and with it into all eight (one).
__device__ __forceinline__ int64_t swz_chunk(int64_t g) { return g ^ (((g >> 3) & 3) << 1); }
__device__ __forceinline__ int4 act_chunk_swz(const int8_t *q, int64_t byte_off) { // byte_off: a multiple of 16
  return *reinterpret_cast<const int4 *>(q + 16 * swz_chunk(byte_off >> 4));
}
__device__ __forceinline__ SmemAct stage_activations(unsigned char *smem, const ActView &a, int blk, bool with_bsum, bool swizzle = false) {
  const int64_t qbytes = a.m * a.k;
  const int64_t dcount = a.m * (a.k / blk);
  int8_t *sq = reinterpret_cast<int8_t *>(smem);
  float *sd = reinterpret_cast<float *>(smem + qbytes);
  int16_t *sb = reinterpret_cast<int16_t *>(smem + qbytes + ((dcount * 4 + 15) & ~(int64_t)15));
  for (int64_t i = threadIdx.x; i < qbytes / 16; i += blockDim.x)
    reinterpret_cast<uint4 *>(sq)[swizzle ? swz_chunk(i) : i] = reinterpret_cast<const uint4 *>(a.q)[i];
  for (int64_t i = threadIdx.x; i < dcount; i += blockDim.x) sd[i] = a.d[i];
  if (with_bsum) {
    const int64_t bwords = a.m * (a.k / 16) / 2; // k/16 is even: pairs of int16
    for (int64_t i = threadIdx.x; i < bwords; i += blockDim.x)
      reinterpret_cast<uint32_t *>(sb)[i] = reinterpret_cast<const uint32_t *>(a.bsum)[i];
  }
  __syncthreads();
  return SmemAct{sq, sd, sb};
}

template <int MT, int R>
__device__ __forceinline__ void reduce_store(float (&acc)[R][MT], int lane, int64_t row0, int64_t n, int m, void *y, int y_dtype,
                                             int64_t ldy) {
#pragma unroll
  for (int r = 0; r < R; r++) {
#pragma unroll
    for (int i = 0; i < MT; i++) {
      const float v = warp_sum(acc[r][i]);
      if (lane == 0 && i < m && row0 + r < n) store_y(y, y_dtype, (int64_t)i * ldy + row0 + r, v);
    }
  }
}

#define XNQ_MATVEC_BOUNDS __launch_bounds__(THREADS, (R >= 4 ? 2 : (MT <= 2 ? 4 : (MT <= 4 ? 3 : 2))))

// ---- Q4_0: one 16-byte chunk = one block (32 codes) ----------------------------------------------
template <int MT, int R>
__global__ void XNQ_MATVEC_BOUNDS matvec_q4_0(WeightView w, ActView a, void *y, int y_dtype, int64_t ldy) {
  extern __shared__ __align__(16) unsigned char smem[];
  const SmemAct sa = stage_activations(smem, a, QK, true);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // persistent over row groups: the activation image is staged once per CTA, not once per WARPS * R rows
  for (int64_t row0 = ((int64_t)blockIdx.x * WARPS + warp) * R; row0 < w.n; row0 += (int64_t)gridDim.x * WARPS * R) {
  const int m = (int)a.m;
  const int64_t k = w.k, nblk = k / QK;
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; r++)
#pragma unroll
    for (int i = 0; i < MT; i++) acc[r][i] = 0.f;

  for (int64_t b = lane; b < nblk; b += 32) {
    uint4 q[R];
    float dw[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int64_t row = min(row0 + r, w.n - 1); // a duplicate row for the ragged tail; never stored
      q[r] = ldg_stream(w.qs + (row * nblk + b) * 16);
      dw[r] = __half2float(w.d[row * w.dstride + b]);
    }
#pragma unroll
    for (int i = 0; i < MT; i++) {
      if (i < m) {
        const int4 alo = *reinterpret_cast<const int4 *>(sa.q + (int64_t)i * k + b * 32);
        const int4 ahi = *reinterpret_cast<const int4 *>(sa.q + (int64_t)i * k + b * 32 + 16);
        const float da = sa.d[(int64_t)i * nblk + b];
        const uint32_t bs2 = *reinterpret_cast<const uint32_t *>(sa.bsum + (int64_t)i * (k / 16) + 2 * b);
        const int bsum = (int)(int16_t)(bs2 & 0xffff) + (int)(int16_t)(bs2 >> 16);
#pragma unroll
        for (int r = 0; r < R; r++) {
          int s = dot16(and4(q[r], 0x0f0f0f0fu), alo, 0);
          s = dot16(and4(shr4(q[r], 4), 0x0f0f0f0fu), ahi, s);
          s -= 8 * bsum; // codes are stored +8
          acc[r][i] += (float)s * dw[r] * da;
        }
      }
    }
  }
  reduce_store<MT, R>(acc, lane, row0, w.n, m, y, y_dtype, ldy);
  }
}

// ---- Q8_0: one 16-byte chunk = half a block -------------------------------------------------------
template <int MT, int R>
__global__ void XNQ_MATVEC_BOUNDS matvec_q8_0(WeightView w, ActView a, void *y, int y_dtype, int64_t ldy) {
  extern __shared__ __align__(16) unsigned char smem[];
  const SmemAct sa = stage_activations(smem, a, QK, false);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // persistent over row groups: the activation image is staged once per CTA, not once per WARPS * R rows
  for (int64_t row0 = ((int64_t)blockIdx.x * WARPS + warp) * R; row0 < w.n; row0 += (int64_t)gridDim.x * WARPS * R) {
  const int m = (int)a.m;
  const int64_t k = w.k, nblk = k / QK, nch = k / 16;
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; r++)
#pragma unroll
    for (int i = 0; i < MT; i++) acc[r][i] = 0.f;

  for (int64_t c = lane; c < nch; c += 32) {
    uint4 q[R];
    float dw[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int64_t row = min(row0 + r, w.n - 1);
      q[r] = ldg_stream(w.qs + row * k + c * 16);
      dw[r] = __half2float(w.d[row * w.dstride + (c >> 1)]);
    }
#pragma unroll
    for (int i = 0; i < MT; i++) {
      if (i < m) {
        const int4 av = *reinterpret_cast<const int4 *>(sa.q + (int64_t)i * k + c * 16);
        const float da = sa.d[(int64_t)i * nblk + (c >> 1)];
#pragma unroll
        for (int r = 0; r < R; r++) acc[r][i] += (float)dot16(q[r], av, 0) * dw[r] * da;
      }
    }
  }
  reduce_store<MT, R>(acc, lane, row0, w.n, m, y, y_dtype, ldy);
  }
}

// ---- Q4_K: 8 lanes per 144-byte super-block (header + 8 chunks of 16 nibble bytes) -----------------
template <int MT, int R>
__global__ void XNQ_MATVEC_BOUNDS matvec_q4k(WeightView w, ActView a, void *y, int y_dtype, int64_t ldy) {
  extern __shared__ __align__(16) unsigned char smem[];
  const SmemAct sa = stage_activations(smem, a, QK_K, true);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // persistent over row groups: the activation image is staged once per CTA, not once per WARPS * R rows
  for (int64_t row0 = ((int64_t)blockIdx.x * WARPS + warp) * R; row0 < w.n; row0 += (int64_t)gridDim.x * WARPS * R) {
  const int m = (int)a.m;
  const int64_t k = w.k, nsb = k / QK_K;
  const int c = lane & 7;      // chunk of the super-block's qs
  const int g = c >> 1;        // 64-element group: sub-blocks 2g (low nibbles) and 2g+1 (high nibbles)
  const int eoff = (c & 1) * 16; // which 16 elements of those sub-blocks
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; r++)
#pragma unroll
    for (int i = 0; i < MT; i++) acc[r][i] = 0.f;

  // With one or two activation rows there are registers to spare: the next iteration's bytes are requested
  // before this iteration's are used, which doubles what a warp keeps in flight (the one-row case at large k
  // is bound by exactly that).
  constexpr bool PREFETCH = MT <= 2;
  uint4 nq[R], nhdr[R];
  if (PREFETCH && (lane >> 3) < nsb) {
#pragma unroll
    for (int r = 0; r < R; r++) {
      const uint8_t *blk = w.qs + (min(row0 + r, w.n - 1) * nsb + (lane >> 3)) * 144;
      nhdr[r] = ldg_stream(blk);
      nq[r] = ldg_stream(blk + 16 + 16 * c);
    }
  }
  for (int64_t sb = lane >> 3; sb < nsb; sb += 4) {
    uint4 q[R];
    float dd[R], dm[R];
    int sc_lo[R], sc_hi[R], mn_lo[R], mn_hi[R];
    uint4 hdrs[R];
    if (PREFETCH) {
#pragma unroll
      for (int r = 0; r < R; r++) q[r] = nq[r], hdrs[r] = nhdr[r];
      if (sb + 4 < nsb) {
#pragma unroll
        for (int r = 0; r < R; r++) {
          const uint8_t *blk = w.qs + (min(row0 + r, w.n - 1) * nsb + sb + 4) * 144;
          nhdr[r] = ldg_stream(blk);
          nq[r] = ldg_stream(blk + 16 + 16 * c);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
      if (!PREFETCH) {
        const int64_t row = min(row0 + r, w.n - 1);
        const uint8_t *blk = w.qs + (row * nsb + sb) * 144;
        hdrs[r] = ldg_stream(blk);
        q[r] = ldg_stream(blk + 16 + 16 * c);
      }
      const uint4 hdr = hdrs[r];
      const __half2 h = *reinterpret_cast<const __half2 *>(&hdr.x);
      dd[r] = __low2float(h);
      dm[r] = __high2float(h);
      const uint32_t f = k4_field(hdr.y, hdr.z, hdr.w, g);
      sc_lo[r] = f & 63;
      sc_hi[r] = (f >> 6) & 63;
      mn_lo[r] = (f >> 12) & 63;
      mn_hi[r] = f >> 18;
    }
    const int64_t kbase = sb * QK_K + 64 * g + eoff;
#pragma unroll
    for (int i = 0; i < MT; i++) {
      if (i < m) {
        const int4 alo = *reinterpret_cast<const int4 *>(sa.q + (int64_t)i * k + kbase);
        const int4 ahi = *reinterpret_cast<const int4 *>(sa.q + (int64_t)i * k + kbase + 32);
        const float da = sa.d[(int64_t)i * nsb + sb];
        const int16_t *bs = sa.bsum + (int64_t)i * (k / 16) + (kbase >> 4);
        const int bs_lo = bs[0], bs_hi = bs[2];
#pragma unroll
        for (int r = 0; r < R; r++) {
          const int s_lo = dot16(and4(q[r], 0x0f0f0f0fu), alo, 0);
          const int s_hi = dot16(and4(shr4(q[r], 4), 0x0f0f0f0fu), ahi, 0);
          const int t1 = sc_lo[r] * s_lo + sc_hi[r] * s_hi;
          const int t2 = mn_lo[r] * bs_lo + mn_hi[r] * bs_hi;
          acc[r][i] += da * (dd[r] * (float)t1 - dm[r] * (float)t2);
        }
      }
    }
  }
  reduce_store<MT, R>(acc, lane, row0, w.n, m, y, y_dtype, ldy);
  }
}

// ---- Q6_K: 4 lanes per super-block; a lane takes 2 ql chunks + 1 qh chunk = 64 codes ---------------
template <int MT, int R>
__global__ void XNQ_MATVEC_BOUNDS matvec_q6k(WeightView w, ActView a, void *y, int y_dtype, int64_t ldy) {
  extern __shared__ __align__(16) unsigned char smem[];
  const SmemAct sa = stage_activations(smem, a, QK_K, true, true);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // persistent over row groups: the activation image is staged once per CTA, not once per WARPS * R rows
  for (int64_t row0 = ((int64_t)blockIdx.x * WARPS + warp) * R; row0 < w.n; row0 += (int64_t)gridDim.x * WARPS * R) {
  const int m = (int)a.m;
  const int64_t k = w.k, nsb = k / QK_K;
  const int u = lane & 3, h = u >> 1, lh = u & 1; // half of the super-block, half of its 32 l-values
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; r++)
#pragma unroll
    for (int i = 0; i < MT; i++) acc[r][i] = 0.f;

  if constexpr (MT >= 8) {
  for (int64_t sb = lane >> 2; sb < nsb; sb += 8) {
    const int64_t kbase = sb * QK_K + 128 * h + 16 * lh; // group gg adds 32*gg
    // The R rows' codes are unpacked first and every activation row's 64 codes are then read from shared memory ONCE for
    // all of them: with the activation loads inside the row loop the kernel was bound by shared-memory bandwidth
    // (one activation byte per multiply-add).
    uint4 code[R][4];
    int sc[R][4];
    float dw[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int64_t row = min(row0 + r, w.n - 1);
      const int64_t blk = row * nsb + sb;
      const uint4 qa = ldg_stream(w.qs + blk * 128 + 64 * h + 16 * lh);
      const uint4 qb = ldg_stream(w.qs + blk * 128 + 64 * h + 32 + 16 * lh);
      const uint4 qh = ldg_stream(w.qh + blk * 64 + 32 * h + 16 * lh);
      const uint2 scw = ldg_stream8(w.sc + blk * 16 + 8 * h);
      dw[r] = __half2float(w.d[row * w.dstride + sb]);
      // 6-bit codes 0..63 of the four 16-element groups (k_quants.rs:1763-1770)
      code[r][0] = or4(and4(qa, 0x0f0f0f0fu), and4(shl4(qh, 4), 0x30303030u));
      code[r][1] = or4(and4(qb, 0x0f0f0f0fu), and4(shl4(qh, 2), 0x30303030u));
      code[r][2] = or4(and4(shr4(qa, 4), 0x0f0f0f0fu), and4(qh, 0x30303030u));
      code[r][3] = or4(and4(shr4(qb, 4), 0x0f0f0f0fu), and4(shr4(qh, 2), 0x30303030u));
      // int8 scales of groups gg: byte index lh + 2*gg of the half's 8 scale bytes
      const uint64_t sc64 = ((uint64_t)scw.y << 32) | scw.x;
#pragma unroll
      for (int gg = 0; gg < 4; gg++) sc[r][gg] = (int)(int8_t)((sc64 >> (8 * (lh + 2 * gg))) & 0xff);
    }
#pragma unroll
    for (int i = 0; i < MT; i++) {
      if (i < m) {
        // the half block's eight 16-sums in one load: group gg of this lane is element lh + 2 gg
        const int4 b8 = *reinterpret_cast<const int4 *>(sa.bsum + (int64_t)i * (k / 16) + sb * 16 + 8 * h);
        const int bw[4] = {b8.x, b8.y, b8.z, b8.w};
        const float da = sa.d[(int64_t)i * nsb + sb];
        int4 av[4];
        int off32[4];
#pragma unroll
        for (int gg = 0; gg < 4; gg++) {
          av[gg] = act_chunk_swz(sa.q, (int64_t)i * k + kbase + 32 * gg);
          off32[gg] = 32 * (int)(int16_t)(bw[gg] >> (16 * lh)); // codes are stored +32
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
          int t = 0;
#pragma unroll
          for (int gg = 0; gg < 4; gg++) t += sc[r][gg] * (dot16(code[r][gg], av[gg], 0) - off32[gg]);
          acc[r][i] += (dw[r] * da) * (float)t;
        }
      }
    }
  }
  } else { // few activation rows: the registers do not hold R rows' codes beside the sums, and the loads are few anyway
  for (int64_t sb = lane >> 2; sb < nsb; sb += 8) {
    const int64_t kbase = sb * QK_K + 128 * h + 16 * lh; // group gg adds 32*gg
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int64_t row = min(row0 + r, w.n - 1);
      const int64_t blk = row * nsb + sb;
      const uint4 qa = ldg_stream(w.qs + blk * 128 + 64 * h + 16 * lh);
      const uint4 qb = ldg_stream(w.qs + blk * 128 + 64 * h + 32 + 16 * lh);
      const uint4 qh = ldg_stream(w.qh + blk * 64 + 32 * h + 16 * lh);
      const uint2 scw = ldg_stream8(w.sc + blk * 16 + 8 * h);
      const float dw = __half2float(w.d[row * w.dstride + sb]);
      // 6-bit codes 0..63 of the four 16-element groups (k_quants.rs:1763-1770)
      uint4 code[4];
      code[0] = or4(and4(qa, 0x0f0f0f0fu), and4(shl4(qh, 4), 0x30303030u));
      code[1] = or4(and4(qb, 0x0f0f0f0fu), and4(shl4(qh, 2), 0x30303030u));
      code[2] = or4(and4(shr4(qa, 4), 0x0f0f0f0fu), and4(qh, 0x30303030u));
      code[3] = or4(and4(shr4(qb, 4), 0x0f0f0f0fu), and4(shr4(qh, 2), 0x30303030u));
      // int8 scales of groups gg: byte index lh + 2*gg of the half's 8 scale bytes
      const uint64_t sc64 = ((uint64_t)scw.y << 32) | scw.x;
      int sc[4];
#pragma unroll
      for (int gg = 0; gg < 4; gg++) sc[gg] = (int)(int8_t)((sc64 >> (8 * (lh + 2 * gg))) & 0xff);
#pragma unroll
      for (int i = 0; i < MT; i++) {
        if (i < m) {
          const int16_t *bs = sa.bsum + (int64_t)i * (k / 16) + (kbase >> 4);
          int t = 0;
#pragma unroll
          for (int gg = 0; gg < 4; gg++) {
            const int4 av = act_chunk_swz(sa.q, (int64_t)i * k + kbase + 32 * gg);
            const int s = dot16(code[gg], av, 0) - 32 * (int)bs[2 * gg]; // codes are stored +32
            t += sc[gg] * s;
          }
          acc[r][i] += (dw * sa.d[(int64_t)i * nsb + sb]) * (float)t;
        }
      }
    }
  }
  }
  reduce_store<MT, R>(acc, lane, row0, w.n, m, y, y_dtype, ldy);
  }
}

template <int MT, int R>
int launch_mt(const WeightView &w, const ActView &a, void *y, int y_dtype, int64_t ldy, cudaStream_t s) {
  const int64_t groups = (w.n + (int64_t)WARPS * R - 1) / ((int64_t)WARPS * R);
  const int blk = (w.dtype == XNQ_Q4_0 || w.dtype == XNQ_Q8_0) ? QK : QK_K;
  const size_t image = smem_act_bytes(a.m, a.k, blk, w.dtype != XNQ_Q8_0);
  const int by_bounds = R >= 4 ? 2 : (MT <= 2 ? 4 : (MT <= 4 ? 3 : 2));
  const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(by_bounds, (220 * 1024) / std::max<size_t>(image + 1024, 1)));
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(groups, (int64_t)g_sms * per_sm));
  switch (w.dtype) {
    case XNQ_Q4_0: {
      const size_t sm = smem_act_bytes(a.m, a.k, QK, true);
      matvec_q4_0<MT, R><<<grid, THREADS, sm, s>>>(w, a, y, y_dtype, ldy);
      break;
    }
    case XNQ_Q8_0: {
      const size_t sm = smem_act_bytes(a.m, a.k, QK, false);
      matvec_q8_0<MT, R><<<grid, THREADS, sm, s>>>(w, a, y, y_dtype, ldy);
      break;
    }
    case XNQ_Q4K: {
      const size_t sm = smem_act_bytes(a.m, a.k, QK_K, true);
      matvec_q4k<MT, R><<<grid, THREADS, sm, s>>>(w, a, y, y_dtype, ldy);
      break;
    }
    case XNQ_Q6K: {
      const size_t sm = smem_act_bytes(a.m, a.k, QK_K, true);
      matvec_q6k<MT, R><<<grid, THREADS, sm, s>>>(w, a, y, y_dtype, ldy);
      break;
    }
    default: return fail(XNQ_ERR_DTYPE, "matvec: dtype %d", w.dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

constexpr size_t MAX_DYN_SMEM = 200 * 1024;

template <int MT, int R>
int init_mt() {
  XNQ_CUDA(cudaFuncSetAttribute(matvec_q4_0<MT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(matvec_q8_0<MT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(matvec_q4k<MT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(matvec_q6k<MT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM));
  return XNQ_OK;
}

} // namespace

// Largest number of activation rows whose quantized image fits the shared-memory budget.
int64_t matvec_rows_per_pass(int wdtype, int64_t k) {
  const int blk = (wdtype == XNQ_Q4_0 || wdtype == XNQ_Q8_0) ? QK : QK_K;
  const bool with_bsum = wdtype != XNQ_Q8_0;
  int64_t rows = MATVEC_MAX_M;
  while (rows > 1 && smem_act_bytes(rows, k, blk, with_bsum) > MAX_DYN_SMEM) rows >>= 1;
  if (smem_act_bytes(rows, k, blk, with_bsum) > MAX_DYN_SMEM) return 0;
  return rows;
}

int launch_matvec(const WeightView &w, const ActView &a, void *y, int y_dtype, int64_t ldy, cudaStream_t s) {
  if (w.n == 0 || a.m == 0) return XNQ_OK;
  if (a.m > MATVEC_MAX_M) return fail(XNQ_ERR_SHAPE, "matvec: m=%lld exceeds %d", (long long)a.m, MATVEC_MAX_M);
  if (a.m == 1) return w.dtype == XNQ_Q4K ? launch_mt<1, 4>(w, a, y, y_dtype, ldy, s) : launch_mt<1, 2>(w, a, y, y_dtype, ldy, s);
  if (a.m == 2) return launch_mt<2, 2>(w, a, y, y_dtype, ldy, s);
  if (a.m <= 4) return launch_mt<4, 2>(w, a, y, y_dtype, ldy, s);
  if (a.m <= 8) return launch_mt<8, 2>(w, a, y, y_dtype, ldy, s);
  return launch_mt<16, 2>(w, a, y, y_dtype, ldy, s);
}

int matvec_init(int device) {
  cudaDeviceProp prop;
  XNQ_CUDA(cudaGetDeviceProperties(&prop, device));
  g_sms = prop.multiProcessorCount;
  int rc;
  if ((rc = init_mt<1, 2>()) != XNQ_OK) return rc;
  if ((rc = init_mt<1, 4>()) != XNQ_OK) return rc;
  if ((rc = init_mt<2, 2>()) != XNQ_OK) return rc;
  if ((rc = init_mt<4, 2>()) != XNQ_OK) return rc;
  if ((rc = init_mt<8, 2>()) != XNQ_OK) return rc;
  if ((rc = init_mt<16, 2>()) != XNQ_OK) return rc;
  return XNQ_OK;
}

} // namespace xnq
