// Weight quantizers on the device: dense f32 [n, k] -> GGUF blocks, bit-identical to the reference's
// host quantizers, which are sequential per sub-block. One thread owns one sub-block and walks it in
// the reference's element order with unfused round-to-nearest arithmetic (every product and sum is
// a separate IEEE operation, as in the Rust source), so the iterative scale searches take the same
// branches and end on the same bits:
//   Q4_0  BlockQ4_0::from_float   k_quants.rs:235-270
//   Q4_K  BlockQ4K::from_float    k_quants.rs:1418-1473, make_qkx1_quants utils.rs:205-254
//   Q6_K  BlockQ6K::from_float    k_quants.rs:1801-1871, make_qx_quants   utils.rs:65-202
//   Q8_0  BlockQ8_0::from_float   k_quants.rs:636-661  (the activation quantizer's kernel)
// This is load-time work (QLinear::from_linear, mod.rs:398-405): throughput matters little, bits do.
#include "xnq_common.cuh"

namespace xnq {
namespace {

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float dvd(float a, float b) { return __fdiv_rn(a, b); }
// nearest_int (utils.rs:3-5): f32::round (half away from zero), then a saturating `as i32` (NaN -> 0)
__device__ __forceinline__ int nearest_int(float v) { return __float2int_rz(roundf(v)); }
__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ unsigned short f16_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ float f16_round(float v) { return __half2float(__float2half_rn(v)); }

template <int N>
__device__ __forceinline__ void load_run(const float *src, float (&x)[N]) {
#pragma unroll
  for (int i = 0; i < N; i += 4) {
    const float4 v = *reinterpret_cast<const float4 *>(src + i);
    x[i] = v.x, x[i + 1] = v.y, x[i + 2] = v.z, x[i + 3] = v.w;
  }
}

// ---- Q4_0: one thread per block of 32 ------------------------------------------------------------
__global__ void __launch_bounds__(128) quantize_q4_0_kernel(const float *x, int64_t nblocks, uint8_t *out) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  float xs[32];
  load_run(x + b * 32, xs);
  float amax = 0.f, mx = 0.f;
#pragma unroll
  for (int j = 0; j < 32; j++) {
    if (amax < fabsf(xs[j])) {
      amax = fabsf(xs[j]);
      mx = xs[j];
    }
  }
  const float d = dvd(mx, -8.0f);
  const float id = d != 0.f ? dvd(1.f, d) : 0.f;
  uint8_t *o = out + b * 18;
  *reinterpret_cast<unsigned short *>(o) = f16_bits(d); // 18-byte blocks start 2-byte aligned
#pragma unroll
  for (int j = 0; j < 16; j += 2) {
    unsigned int pair = 0;
#pragma unroll
    for (int t = 0; t < 2; t++) {
      // `as u8` saturates: negative -> 0, above 255 -> 255, NaN -> 0; then min(15)
      const float f0 = add(mul(xs[j + t], id), 8.5f), f1 = add(mul(xs[16 + j + t], id), 8.5f);
      const int i0 = min(max(__float2int_rz(f0), 0), 15), i1 = min(max(__float2int_rz(f1), 0), 15);
      pair |= (unsigned int)(i0 | (i1 << 4)) << (8 * t);
    }
    *reinterpret_cast<unsigned short *>(o + 2 + j) = (unsigned short)pair;
  }
}

// ---- Q4_K: one thread per sub-block of 32, eight neighbouring threads per super-block -------------
__device__ __forceinline__ void make_qkx1(const float (&x)[32], float &scale_out, float &min_out) {
  constexpr int nmax = 15, ntry = 5;
  unsigned char l[32];
#pragma unroll
  for (int i = 0; i < 32; i++) l[i] = 0;
  float mn = x[0], mx = x[0];
#pragma unroll
  for (int i = 1; i < 32; i++) {
    if (x[i] < mn) mn = x[i];
    if (x[i] > mx) mx = x[i];
  }
  if (mx == mn) {
    scale_out = 0.f, min_out = 0.f;
    return;
  }
  if (mn > 0.f) mn = 0.f;
  float iscale = dvd((float)nmax, sub(mx, mn));
  float scale = dvd(1.0f, iscale);
  for (int t = 0; t < ntry; t++) {
    float sumlx = 0.f;
    int suml2 = 0;
    bool changed = false;
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const float xm = sub(x[i], mn);
      const int li = clampi(nearest_int(mul(iscale, xm)), 0, nmax);
      if ((unsigned char)li != l[i]) {
        l[i] = (unsigned char)li;
        changed = true;
      }
      sumlx = add(sumlx, mul(xm, (float)li));
      suml2 += li * li;
    }
    scale = dvd(sumlx, (float)suml2);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) sum = add(sum, sub(x[i], mul(scale, (float)l[i])));
    mn = dvd(sum, 32.0f);
    if (mn > 0.f) mn = 0.f;
    iscale = dvd(1.0f, scale);
    if (!changed) break;
  }
  scale_out = scale;
  min_out = -mn;
}

__global__ void __launch_bounds__(128) quantize_q4k_kernel(const float *x, int64_t nsub, uint8_t *out) {
  const int64_t sub_id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; // nsub is a multiple of 8 and blockDim of 8: super-blocks never straddle
  const bool live = sub_id < nsub;
  const int j = threadIdx.x & 7;
  float xs[32];
  float scale = 0.f, mn = 0.f;
  if (live) {
    load_run(x + sub_id * 32, xs);
    make_qkx1(xs, scale, mn);
  } else {
#pragma unroll
    for (int i = 0; i < 32; i++) xs[i] = 0.f;
  }
  float max_scale = scale, max_min = mn;
#pragma unroll
  for (int off = 1; off < 8; off <<= 1) {
    max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, off));
    max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, off));
  }
  max_scale = fmaxf(max_scale, 0.f), max_min = fmaxf(max_min, 0.f); // the reference's running maxima start at 0
  const float inv_scale = max_scale > 0.f ? dvd(63.0f, max_scale) : 0.f;
  const float inv_min = max_min > 0.f ? dvd(63.0f, max_min) : 0.f;
  const int ls = min(nearest_int(mul(inv_scale, scale)), 63) & 0xff; // `as u8` of a value in 0..63
  const int lm = min(nearest_int(mul(inv_min, mn)), 63) & 0xff;
  const float d16 = f16_round(dvd(max_scale, 63.0f)), dmin16 = f16_round(dvd(max_min, 63.0f));
  // codes of this sub-block with the 6-bit scale and min as they will be read back
  const float d = mul(d16, (float)(ls & 63));
  unsigned int packed[8]; // one code per byte
#pragma unroll
  for (int w = 0; w < 8; w++) packed[w] = 0;
  if (d != 0.f) {
    const float dm = mul(dmin16, (float)(lm & 63));
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const int lv = clampi(nearest_int(dvd(add(xs[i], dm), d)), 0, 15);
      packed[i >> 2] |= (unsigned int)lv << (8 * (i & 3));
    }
  }
  // the 12 scale bytes, assembled by every thread from its neighbours' 6-bit values (k_quants.rs:1434-1445)
  unsigned int sc[3] = {0, 0, 0};
#pragma unroll
  for (int t = 0; t < 8; t++) {
    const unsigned int s6 = (unsigned int)__shfl_sync(0xffffffffu, ls, (threadIdx.x & 24) | t) & 63u;
    const unsigned int m6 = (unsigned int)__shfl_sync(0xffffffffu, lm, (threadIdx.x & 24) | t) & 63u;
    auto put = [&](int byte, unsigned int v) { sc[byte >> 2] |= v << (8 * (byte & 3)); };
    if (t < 4) {
      put(t, s6);
      put(t + 4, m6);
    } else {
      put(t + 4, (s6 & 0xF) | ((m6 & 0xF) << 4));
      put(t - 4, (s6 >> 4) << 6);
      put(t, (m6 >> 4) << 6);
    }
  }
  // low nibbles: sub-block 2c, high nibbles: sub-block 2c+1, byte by byte
  unsigned int outw[8];
#pragma unroll
  for (int w = 0; w < 8; w++) outw[w] = packed[w] | (__shfl_down_sync(0xffffffffu, packed[w], 1) << 4);
  if (!live) return;
  uint8_t *blk = out + (sub_id >> 3) * 144;
  if (j == 0) {
    uint4 h;
    h.x = (unsigned int)f16_bits(dvd(max_scale, 63.0f)) | ((unsigned int)f16_bits(dvd(max_min, 63.0f)) << 16);
    h.y = sc[0], h.z = sc[1], h.w = sc[2];
    *reinterpret_cast<uint4 *>(blk) = h;
  }
  if ((j & 1) == 0) {
    uint4 *q = reinterpret_cast<uint4 *>(blk + 16 + (j >> 1) * 32);
    q[0] = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    q[1] = make_uint4(outw[4], outw[5], outw[6], outw[7]);
  }
}

// ---- Q6_K: one thread per group of 16, sixteen neighbouring threads per super-block ---------------
// make_qx_quants(n = 16, nmax = 32, rmse_type = 1): weights w = x^2, returns before the final grid search
__device__ __forceinline__ float make_qx_16(const float (&x)[16], signed char (&ls)[16]) {
  constexpr int nmax = 32;
  float mx = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; i++) {
    const float ax = fabsf(x[i]);
    if (ax > amax) {
      amax = ax;
      mx = x[i];
    }
  }
  if (amax == 0.f) {
#pragma unroll
    for (int i = 0; i < 16; i++) ls[i] = 0;
    return 0.f;
  }
  const float iscale = dvd(-(float)nmax, mx);
  float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; i++) {
    const int l = clampi(nearest_int(mul(iscale, x[i])), -nmax, nmax - 1);
    ls[i] = (signed char)(l + nmax);
    const float w = mul(x[i], x[i]), lf = (float)l;
    sumlx = add(sumlx, mul(mul(w, x[i]), lf));
    suml2 = add(suml2, mul(mul(w, lf), lf));
  }
  float scale = dvd(sumlx, suml2);
  float best = mul(scale, sumlx);
  for (int itry = 0; itry < 3; itry++) {
    const float isc = dvd(1.0f, scale);
    float slx = 0.f, sl2 = 0.f;
    bool changed = false;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const int l = clampi(nearest_int(mul(isc, x[i])), -nmax, nmax - 1);
      if (l + nmax != (int)ls[i]) changed = true;
      const float w = mul(x[i], x[i]), lf = (float)l;
      slx = add(slx, mul(mul(w, x[i]), lf));
      sl2 = add(sl2, mul(mul(w, lf), lf));
    }
    if (!changed || sl2 == 0.f || mul(slx, slx) <= mul(best, sl2)) break;
#pragma unroll
    for (int i = 0; i < 16; i++) ls[i] = (signed char)(nmax + clampi(nearest_int(mul(isc, x[i])), -nmax, nmax - 1));
    sumlx = slx, suml2 = sl2;
    scale = dvd(sumlx, suml2);
    best = mul(scale, sumlx);
  }
  for (int itry = 0; itry < 5; itry++) {
    int n_changed = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const float w = mul(x[i], x[i]);
      const int l = (int)ls[i] - nmax;
      float slx = sub(sumlx, mul(mul(w, x[i]), (float)l));
      if (slx > 0.f) {
        float sl2 = sub(suml2, mul(mul(w, (float)l), (float)l));
        const int new_l = clampi(nearest_int(dvd(mul(x[i], sl2), slx)), -nmax, nmax - 1);
        if (new_l != l) {
          slx = add(slx, mul(mul(w, x[i]), (float)new_l));
          sl2 = add(sl2, mul(mul(w, (float)new_l), (float)new_l));
          if (sl2 > 0.f && mul(mul(slx, slx), suml2) > mul(mul(sumlx, sumlx), sl2)) {
            ls[i] = (signed char)(nmax + new_l);
            sumlx = slx, suml2 = sl2;
            scale = dvd(sumlx, suml2);
            best = mul(scale, sumlx);
            n_changed++;
          }
        }
      }
    }
    if (n_changed == 0) break;
  }
  return scale;
}

__global__ void __launch_bounds__(128) quantize_q6k_kernel(const float *x, int64_t ngroups, uint8_t *out) {
  __shared__ unsigned char codes[128 / 16][256]; // one row per super-block of this CTA
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; // ngroups is a multiple of 16, as is blockDim
  const bool live = gid < ngroups;
  const int g = threadIdx.x & 15, sbl = threadIdx.x >> 4;
  float xs[16];
  signed char ls[16];
  float scale = 0.f;
  if (live) {
    load_run(x + gid * 16, xs);
    scale = make_qx_16(xs, ls);
  } else {
#pragma unroll
    for (int i = 0; i < 16; i++) xs[i] = 0.f, ls[i] = 0;
  }
  // the first group with the largest |scale| provides the signed maximum (strict >, in group order)
  float max_scale = 0.f, max_abs = 0.f;
#pragma unroll
  for (int t = 0; t < 16; t++) {
    const float s = __shfl_sync(0xffffffffu, scale, (threadIdx.x & 16) | t);
    if (fabsf(s) > max_abs) {
      max_abs = fabsf(s);
      max_scale = s;
    }
  }
  const float iscale = dvd(-128.f, max_scale);
  const float dfull = dvd(1.0f, iscale);
  const float d16 = f16_round(dfull);
  const int sc8 = max(min(nearest_int(mul(iscale, scale)), 127), -128);
  const float d = mul(d16, (float)sc8);
  if (d != 0.f) {
#pragma unroll
    for (int i = 0; i < 16; i++) ls[i] = (signed char)(clampi(nearest_int(dvd(xs[i], d)), -32, 31) + 32);
  }
#pragma unroll
  for (int i = 0; i < 16; i += 4)
    *reinterpret_cast<unsigned int *>(&codes[sbl][16 * g + i]) =
        (unsigned int)(unsigned char)ls[i] | ((unsigned int)(unsigned char)ls[i + 1] << 8) | ((unsigned int)(unsigned char)ls[i + 2] << 16) |
        ((unsigned int)(unsigned char)ls[i + 3] << 24);
  __syncthreads();
  if (!live) return;
  uint8_t *blk = out + (gid >> 4) * 210; // 210-byte blocks: 2-byte aligned only
  // thread g packs 4 columns of one 128-half: half h = g / 8, columns li = 4 * (g % 8) ..
  const int h = g >> 3, li0 = (g & 7) * 4;
  const unsigned char *l = &codes[sbl][128 * h];
  unsigned short ql_a[2], ql_b[2], qh2[2];
#pragma unroll
  for (int p = 0; p < 2; p++) {
    unsigned int a = 0, b = 0, q = 0;
#pragma unroll
    for (int t = 0; t < 2; t++) {
      const int li = li0 + 2 * p + t;
      const unsigned int l0 = l[li], l1 = l[li + 32], l2 = l[li + 64], l3 = l[li + 96];
      a |= ((l0 & 0xF) | ((l2 & 0xF) << 4)) << (8 * t);
      b |= ((l1 & 0xF) | ((l3 & 0xF) << 4)) << (8 * t);
      q |= ((l0 >> 4) | ((l1 >> 4) << 2) | ((l2 >> 4) << 4) | ((l3 >> 4) << 6)) << (8 * t);
    }
    ql_a[p] = (unsigned short)a, ql_b[p] = (unsigned short)b, qh2[p] = (unsigned short)q;
  }
#pragma unroll
  for (int p = 0; p < 2; p++) {
    *reinterpret_cast<unsigned short *>(blk + 64 * h + li0 + 2 * p) = ql_a[p];
    *reinterpret_cast<unsigned short *>(blk + 64 * h + 32 + li0 + 2 * p) = ql_b[p];
    *reinterpret_cast<unsigned short *>(blk + 128 + 32 * h + li0 + 2 * p) = qh2[p];
  }
  blk[192 + g] = (uint8_t)(signed char)sc8;
  if (g == 0) *reinterpret_cast<unsigned short *>(blk + 208) = f16_bits(dfull);
}

} // namespace

int launch_quantize_weight(int dtype, const float *x, int64_t n, int64_t k, void *blocks, cudaStream_t s) {
  const int64_t elems = n * k;
  if (elems == 0) return XNQ_OK;
  switch (dtype) {
    case XNQ_Q4_0: {
      const int64_t nb = elems / 32;
      quantize_q4_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, s>>>(x, nb, static_cast<uint8_t *>(blocks));
      break;
    }
    case XNQ_Q8_0: return launch_quantize_act_blocks(XNQ_Q8_0, x, XNQ_F32, n, k, k, blocks, s);
    case XNQ_Q4K: {
      const int64_t ns = elems / 32;
      quantize_q4k_kernel<<<(unsigned)((ns + 127) / 128), 128, 0, s>>>(x, ns, static_cast<uint8_t *>(blocks));
      break;
    }
    case XNQ_Q6K: {
      const int64_t ng = elems / 16;
      quantize_q6k_kernel<<<(unsigned)((ng + 127) / 128), 128, 0, s>>>(x, ng, static_cast<uint8_t *>(blocks));
      break;
    }
    default: return fail(XNQ_ERR_DTYPE, "quantize_weight: dtype %d is not a weight format", dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

} // namespace xnq
