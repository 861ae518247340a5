// The GGML formats beyond the four of the benchmark configurations: Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K as weight
// formats and Q8_1 as an activation format (xn-core/src/quantized/k_quants.rs:100-186 block layouts, 307-610 the
// 32-element formats, 834-878 Q8_1, 880-1316 Q2_K / Q3_K, 1507-1722 Q5_K).
//
// Real GGUF files mix types, so a handle must be able to hold any of them; none of these formats is on the measured path.
// They are therefore kept on the device exactly as in the file (canonical blocks, no re-layout) and served by one plain
// kernel per operation:
//   to_float   one thread per element, the reference's arithmetic operation for operation (bit-identical results);
//   matmul     activations are quantized to the canonical blocks of the format's VecDotType (Q8_0, Q8_1 or Q8_K, by the
//              same quantizers that xnq_quantize_act exposes, byte-identical to the reference's), then one warp per
//              weight row, lane l taking blocks l, l + 32, ...: each block's integer sums and its scaling in f32 are
//              exactly the reference's, the block contributions are added lane-wise and then across the warp (the one
//              difference from the reference's serial sum; within 2e-3 under its own metric). All activation rows are
//              served by the same warp in turn, so the weight is read from DRAM once.
// HBM-bound streaming kernels in the style of the four main formats would be the next step for any of these formats that
// turns out to matter.
#include "xnq_common.cuh"
#include "xnq_quantize_act.cuh"
#include "xnq_unpack.cuh"

namespace xnq {
namespace {

constexpr int TPB = 256;

__device__ __forceinline__ uint32_t ld16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); } // blocks are 2-byte aligned
__device__ __forceinline__ uint32_t ld32(const uint8_t *p) { return ld16(p) | (ld16(p + 2) << 16); }
__device__ __forceinline__ float ldh(const uint8_t *p) { return __half2float(__ushort_as_half((unsigned short)ld16(p))); }
__device__ __forceinline__ float ldf(const uint8_t *p) { return __uint_as_float(ld32(p)); }
__device__ __forceinline__ int ldi8(const uint8_t *p) { return (int)(int8_t)*p; }
__device__ __forceinline__ int ldi16(const uint8_t *p) { return (int)(int16_t)ld16(p); }

// 6-bit (scale, min) pair j of the 12 packed bytes of a Q4_K / Q5_K block (utils.rs:53-63)
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int &sc, int &mn) {
  if (j < 4) {
    sc = q[j] & 63;
    mn = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}
// the sixteen 6-bit scales of a Q3_K block (k_quants.rs:1122-1127): scale s as an unsigned byte, before the -32
__device__ __forceinline__ int q3k_scale(const uint8_t *packed, int s) {
  const uint32_t a0 = ld32(packed), a1 = ld32(packed + 4), tmp = ld32(packed + 8);
  const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu;
  uint32_t w;
  switch (s >> 2) {
    case 0: w = (a0 & kmask2) | (((tmp) & kmask1) << 4); break;
    case 1: w = (a1 & kmask2) | (((tmp >> 2) & kmask1) << 4); break;
    case 2: w = ((a0 >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4); break;
    default: w = ((a1 >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4); break;
  }
  return (int)(int8_t)((w >> (8 * (s & 3))) & 0xff);
}

// ---- to_float: element j of a block, the reference's expression with every operation rounded separately --------------
__device__ __forceinline__ float deq_q4_1(const uint8_t *b, int j) { // {f16 d; f16 m; u8 qs[16]}, k_quants.rs:379-399
  const int q = j < 16 ? (b[4 + j] & 0x0F) : (b[4 + j - 16] >> 4);
  return __fadd_rn(__fmul_rn((float)q, ldh(b)), ldh(b + 2));
}
__device__ __forceinline__ int code_q5(uint32_t qh, const uint8_t *qs, int j) { // 5-bit code of element j (k_quants.rs:489-497)
  return j < 16 ? ((qs[j] & 0x0F) | (((qh >> j) << 4) & 0x10)) : ((qs[j - 16] >> 4) | ((qh >> (j - 16 + 12)) & 0x10));
}
__device__ __forceinline__ float deq_q5_0(const uint8_t *b, int j) { // {f16 d; u8 qh[4]; u8 qs[16]}, k_quants.rs:478-502
  return __fmul_rn((float)(code_q5(ld32(b + 2), b + 6, j) - 16), ldh(b));
}
__device__ __forceinline__ float deq_q5_1(const uint8_t *b, int j) { // {f16 d; f16 m; u8 qh[4]; u8 qs[16]}, k_quants.rs:586-612
  return __fadd_rn(__fmul_rn((float)code_q5(ld32(b + 4), b + 8, j), ldh(b)), ldh(b + 2));
}
__device__ __forceinline__ float deq_q2k(const uint8_t *b, int j) { // {u8 scales[16]; u8 qs[64]; f16 d; f16 dmin}, k_quants.rs:1014-1056
  const int half = j >> 7, jj = j & 127, sh = jj >> 5, l = jj & 31;
  const int sc = b[8 * half + 2 * sh + (l >> 4)];
  const float dl = __fmul_rn(ldh(b + 80), (float)(sc & 0xF)), ml = __fmul_rn(ldh(b + 82), (float)(sc >> 4));
  const int q = (b[16 + 32 * half + l] >> (2 * sh)) & 3;
  return __fsub_rn(__fmul_rn(dl, (float)q), ml);
}
__device__ __forceinline__ int code_q3k(const uint8_t *b, int j) { // signed code of element j (k_quants.rs:1290-1300)
  const int half = j >> 7, jj = j & 127, sh = jj >> 5, l = jj & 31;
  const int q = (b[32 + 32 * half + l] >> (2 * sh)) & 3;
  return q - ((b[l] & (1 << (4 * half + sh))) ? 0 : 4);
}
__device__ __forceinline__ float deq_q3k(const uint8_t *b, int j) { // {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d}, k_quants.rs:1260-1313
  const float dl = __fmul_rn(ldh(b + 108), __fsub_rn((float)q3k_scale(b + 96, j >> 4), 32.0f));
  return __fmul_rn(dl, (float)code_q3k(b, j));
}
__device__ __forceinline__ int code_q5k(const uint8_t *b, int j) { // 5-bit code of element j (k_quants.rs:1700-1709)
  const int c = j >> 6, jj = j & 63, l = jj & 31, hi = jj >> 5;
  const int q = hi ? (b[48 + 32 * c + l] >> 4) : (b[48 + 32 * c + l] & 0xF);
  return q + ((b[16 + l] & (1 << (2 * c + hi))) ? 16 : 0);
}
__device__ __forceinline__ float deq_q5k(const uint8_t *b, int j) { // {f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]}, k_quants.rs:1684-1718
  int sc, mn;
  scale_min_k4(j >> 5, b + 4, sc, mn);
  const float d1 = __fmul_rn(ldh(b), (float)sc), m1 = __fmul_rn(ldh(b + 2), (float)mn);
  return __fsub_rn(__fmul_rn(d1, (float)code_q5k(b, j)), m1); // (ql + 16) is exact in f32, as in the reference's (ql as f32 + to_add)
}

template <typename T>
__device__ __forceinline__ T cast_to(float v);
template <>
__device__ __forceinline__ float cast_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_to<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_to<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(TPB) generic_dequantize_kernel(int dtype, const uint8_t *blocks, int64_t total, int bs, int ts, T *out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= total) return;
  const uint8_t *b = blocks + (i / bs) * ts;
  const int j = (int)(i % bs);
  float v;
  switch (dtype) {
    case XNQ_Q4_1: v = deq_q4_1(b, j); break;
    case XNQ_Q5_0: v = deq_q5_0(b, j); break;
    case XNQ_Q5_1: v = deq_q5_1(b, j); break;
    case XNQ_Q2K: v = deq_q2k(b, j); break;
    case XNQ_Q3K: v = deq_q3k(b, j); break;
    default: v = deq_q5k(b, j); break;
  }
  out[i] = cast_to<T>(v);
}

// ---- Q8_1 activation quantizer (k_quants.rs:847-873): one thread per 32-element block -------------------------------
template <typename XT>
__global__ void __launch_bounds__(TPB) quantize_q8_1_kernel(const XT *x, int64_t m, int64_t k, int64_t ldx, uint8_t *dst) {
  const int64_t nb_row = k / 32, i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= m * nb_row) return;
  const int64_t r = i / nb_row, bi = i % nb_row;
  float v[32];
#pragma unroll
  for (int c = 0; c < 4; c++) load8(x + r * ldx + bi * 32 + 8 * c, v + 8 * c);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(v[j])); // fmaxf ignores a NaN operand, as f32::max does
  const float d = __fdiv_rn(amax, 127.0f), id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
  const __half dh = __float2half_rn(d);
  uint8_t *b = dst + i * 36;
  int sum = 0;
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const int q = round_away_sat_i8(__fmul_rn(v[j], id));
    b[4 + j] = (uint8_t)(int8_t)q;
    sum += q;
  }
  // s = f16(sum) * d as f16 values: both widened to f32, multiplied, the product rounded back to f16
  const __half sh = __float2half_rn(__fmul_rn(__half2float(__float2half_rn((float)sum)), __half2float(dh)));
  *reinterpret_cast<uint16_t *>(b) = __half_as_ushort(dh);
  *reinterpret_cast<uint16_t *>(b + 2) = __half_as_ushort(sh);
}

// ---- dots: one weight block against the matching activation block(s), exactly the reference's arithmetic -------------
// 32-element formats: a = the activation block (Q8_0 {f16 d; i8 qs[32]} or Q8_1 {f16 d; f16 s; i8 qs[32]})
__device__ __forceinline__ float dot_q4_1(const uint8_t *w, const uint8_t *a) { // k_quants.rs:328-339
  int sumi = 0;
#pragma unroll
  for (int j = 0; j < 16; j++) sumi += (w[4 + j] & 0x0F) * ldi8(a + 4 + j) + (w[4 + j] >> 4) * ldi8(a + 4 + j + 16);
  return __fadd_rn(__fmul_rn(__fmul_rn((float)sumi, ldh(w)), ldh(a)), __fmul_rn(ldh(w + 2), ldh(a + 2)));
}
__device__ __forceinline__ float dot_q5_0(const uint8_t *w, const uint8_t *a) { // k_quants.rs:423-436
  const uint32_t qh = ld32(w + 2);
  int sumi = 0;
#pragma unroll
  for (int j = 0; j < 32; j++) sumi += (code_q5(qh, w + 6, j) - 16) * ldi8(a + 2 + j);
  return __fmul_rn(__fmul_rn((float)sumi, ldh(w)), ldh(a));
}
__device__ __forceinline__ float dot_q5_1(const uint8_t *w, const uint8_t *a) { // k_quants.rs:529-541
  const uint32_t qh = ld32(w + 4);
  int sumi = 0;
#pragma unroll
  for (int j = 0; j < 32; j++) sumi += code_q5(qh, w + 8, j) * ldi8(a + 4 + j);
  return __fadd_rn(__fmul_rn(__fmul_rn((float)sumi, ldh(w)), ldh(a)), __fmul_rn(ldh(w + 2), ldh(a + 2)));
}
// 256-element formats: a = BlockQ8K {f32 d; i8 qs[256]; i16 bsums[16]}
__device__ __forceinline__ float dot_q2k(const uint8_t *w, const uint8_t *a) { // k_quants.rs:904-945
  int summs = 0;
#pragma unroll
  for (int j = 0; j < 16; j++) summs += ldi16(a + 260 + 2 * j) * (w[j] >> 4);
  const float ad = ldf(a), dall = __fmul_rn(ad, ldh(w + 80)), dmin = __fmul_rn(ad, ldh(w + 82));
  int isum = 0;
  for (int g = 0; g < 16; g++) { // group g: 16 elements; half = g / 8, shift pair = (g % 8) / 2, part = g % 2
    const int half = g >> 3, sh = (g & 7) >> 1, part = g & 1;
    const uint8_t *q2 = w + 16 + 32 * half + 16 * part;
    const uint8_t *q8 = a + 4 + 128 * half + 32 * sh + 16 * part;
    int isuml = 0;
#pragma unroll
    for (int l = 0; l < 16; l++) isuml += ldi8(q8 + l) * ((q2[l] >> (2 * sh)) & 3);
    isum += (w[g] & 0xF) * isuml;
  }
  return __fsub_rn(__fmul_rn(dall, (float)isum), __fmul_rn(dmin, (float)summs));
}
__device__ __forceinline__ float dot_q3k(const uint8_t *w, const uint8_t *a) { // k_quants.rs:1087-1176: eight f32 lanes per block, added here
  int aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int s = 0; s < 16; s++) {
    const int scale = q3k_scale(w + 96, s) - 32;
#pragma unroll
    for (int e = 0; e < 16; e++) aux32[e & 7] += scale * (ldi8(a + 4 + 16 * s + e) * code_q3k(w, 16 * s + e));
  }
  const float d = __fmul_rn(ldh(w + 108), ldf(a));
  float t = 0.f;
#pragma unroll
  for (int l = 0; l < 8; l++) t = __fadd_rn(t, __fmul_rn(d, (float)aux32[l]));
  return t;
}
__device__ __forceinline__ float dot_q5k(const uint8_t *w, const uint8_t *a) { // k_quants.rs:1540-1604
  int aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int sumi = 0;
  for (int s = 0; s < 8; s++) {
    int sc, mn;
    scale_min_k4(s, w + 4, sc, mn);
    sumi += (ldi16(a + 260 + 4 * s) + ldi16(a + 260 + 4 * s + 2)) * mn;
#pragma unroll
    for (int e = 0; e < 32; e++) aux32[e & 7] += sc * (ldi8(a + 4 + 32 * s + e) * code_q5k(w, 32 * s + e));
  }
  const float ad = ldf(a), d = __fmul_rn(ldh(w), ad), dmin = __fmul_rn(ldh(w + 2), ad);
  float t = 0.f;
#pragma unroll
  for (int l = 0; l < 8; l++) t = __fadd_rn(t, __fmul_rn(d, (float)aux32[l]));
  return __fsub_rn(t, __fmul_rn(dmin, (float)sumi));
}

// One warp per weight row; lane l takes blocks l, l + 32, ...; activation rows in turn.
template <int DT>
__global__ void __launch_bounds__(TPB) generic_matmul_kernel(const uint8_t *w, const uint8_t *act, int64_t n, int64_t m, int nblk, int wts, int ats, void *y,
                                                             int y_dtype, int64_t ldy) {
  const int64_t row = blockIdx.x * (int64_t)(TPB / 32) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const uint8_t *wr = w + row * (int64_t)nblk * wts;
  for (int64_t r = 0; r < m; r++) {
    const uint8_t *ar = act + r * (int64_t)nblk * ats;
    float sum = 0.f;
    for (int b = lane; b < nblk; b += 32) {
      const uint8_t *wb = wr + (int64_t)b * wts, *ab = ar + (int64_t)b * ats;
      float v;
      if (DT == XNQ_Q4_1) v = dot_q4_1(wb, ab);
      else if (DT == XNQ_Q5_0) v = dot_q5_0(wb, ab);
      else if (DT == XNQ_Q5_1) v = dot_q5_1(wb, ab);
      else if (DT == XNQ_Q2K) v = dot_q2k(wb, ab);
      else if (DT == XNQ_Q3K) v = dot_q3k(wb, ab);
      else v = dot_q5k(wb, ab);
      sum += v;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) {
      const int64_t idx = r * ldy + row;
      if (y_dtype == XNQ_F32) static_cast<float *>(y)[idx] = sum;
      else if (y_dtype == XNQ_F16) static_cast<__half *>(y)[idx] = __float2half_rn(sum);
      else static_cast<__nv_bfloat16 *>(y)[idx] = __float2bfloat16_rn(sum);
    }
  }
}

inline unsigned grid_for(int64_t work, int per) { return (unsigned)((work + per - 1) / per); }

} // namespace

bool is_generic_dtype(int dt) { return dt == XNQ_Q4_1 || dt == XNQ_Q5_0 || dt == XNQ_Q5_1 || dt == XNQ_Q2K || dt == XNQ_Q3K || dt == XNQ_Q5K; }

int launch_generic_dequantize(const WeightView &w, int out_dtype, void *dst, cudaStream_t s) {
  if (w.n == 0) return XNQ_OK;
  const int64_t total = w.n * w.k;
  const int bs = block_size(w.dtype), ts = type_size(w.dtype);
  const unsigned g = grid_for(total, TPB);
  switch (out_dtype) {
    case XNQ_F32: generic_dequantize_kernel<float><<<g, TPB, 0, s>>>(w.dtype, w.qs, total, bs, ts, static_cast<float *>(dst)); break;
    case XNQ_F16: generic_dequantize_kernel<__half><<<g, TPB, 0, s>>>(w.dtype, w.qs, total, bs, ts, static_cast<__half *>(dst)); break;
    case XNQ_BF16: generic_dequantize_kernel<__nv_bfloat16><<<g, TPB, 0, s>>>(w.dtype, w.qs, total, bs, ts, static_cast<__nv_bfloat16 *>(dst)); break;
    default: return fail(XNQ_ERR_DTYPE, "dequantize: output dtype %d is not f32/f16/bf16", out_dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int launch_quantize_q8_1(const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx, void *dst, cudaStream_t s) {
  if (m == 0) return XNQ_OK;
  const unsigned g = grid_for(m * (k / 32), TPB);
  uint8_t *d = static_cast<uint8_t *>(dst);
  switch (x_dtype) {
    case XNQ_F32: quantize_q8_1_kernel<float><<<g, TPB, 0, s>>>(static_cast<const float *>(x), m, k, ldx, d); break;
    case XNQ_F16: quantize_q8_1_kernel<__half><<<g, TPB, 0, s>>>(static_cast<const __half *>(x), m, k, ldx, d); break;
    case XNQ_BF16: quantize_q8_1_kernel<__nv_bfloat16><<<g, TPB, 0, s>>>(static_cast<const __nv_bfloat16 *>(x), m, k, ldx, d); break;
    default: return fail(XNQ_ERR_DTYPE, "quantize_act: activation dtype %d", x_dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

size_t generic_workspace_bytes(const WeightView &w, int64_t m) {
  const int adt = act_dtype_for(w.dtype);
  return ((size_t)m * (size_t)(w.k / block_size(adt)) * (size_t)type_size(adt) + 255) & ~(size_t)255;
}

// y[m, n] = x[m, k] . W^T for a weight held as canonical blocks; workspace: generic_workspace_bytes(w, m)
int launch_generic_matmul(const WeightView &w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy, void *workspace,
                          cudaStream_t s) {
  const int adt = act_dtype_for(w.dtype);
  // the reference's dots of the 32-element formats refuse an odd number of blocks (k_quants.rs:322-325, 413-415, 523-526)
  if (block_size(w.dtype) == 32 && (w.k / 32) % 2) return fail(XNQ_ERR_SHAPE, "matmul_t: k = %lld is not divisible by 64 (an even number of 32-value blocks)", (long long)w.k);
  int rc = adt == XNQ_Q8_1 ? launch_quantize_q8_1(x, x_dtype, m, w.k, ldx, workspace, s) : launch_quantize_act_blocks(adt, x, x_dtype, m, w.k, ldx, workspace, s);
  if (rc != XNQ_OK) return rc;
  const int nblk = (int)(w.k / block_size(w.dtype)), wts = type_size(w.dtype), ats = type_size(adt);
  const unsigned g = grid_for(w.n, TPB / 32);
  const uint8_t *act = static_cast<const uint8_t *>(workspace);
  profile_mark(s, true);
  switch (w.dtype) {
    case XNQ_Q4_1: generic_matmul_kernel<XNQ_Q4_1><<<g, TPB, 0, s>>>(w.qs, act, w.n, m, nblk, wts, ats, y, y_dtype, ldy); break;
    case XNQ_Q5_0: generic_matmul_kernel<XNQ_Q5_0><<<g, TPB, 0, s>>>(w.qs, act, w.n, m, nblk, wts, ats, y, y_dtype, ldy); break;
    case XNQ_Q5_1: generic_matmul_kernel<XNQ_Q5_1><<<g, TPB, 0, s>>>(w.qs, act, w.n, m, nblk, wts, ats, y, y_dtype, ldy); break;
    case XNQ_Q2K: generic_matmul_kernel<XNQ_Q2K><<<g, TPB, 0, s>>>(w.qs, act, w.n, m, nblk, wts, ats, y, y_dtype, ldy); break;
    case XNQ_Q3K: generic_matmul_kernel<XNQ_Q3K><<<g, TPB, 0, s>>>(w.qs, act, w.n, m, nblk, wts, ats, y, y_dtype, ldy); break;
    case XNQ_Q5K: generic_matmul_kernel<XNQ_Q5K><<<g, TPB, 0, s>>>(w.qs, act, w.n, m, nblk, wts, ats, y, y_dtype, ldy); break;
    default: return fail(XNQ_ERR_DTYPE, "matmul_t: dtype %d", w.dtype);
  }
  profile_mark(s, false);
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int generic_init(int) { // kernels are loaded before any stream capture
  cudaFuncAttributes fa;
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_dequantize_kernel<float>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_dequantize_kernel<__half>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_dequantize_kernel<__nv_bfloat16>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_q8_1_kernel<float>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_q8_1_kernel<__half>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_q8_1_kernel<__nv_bfloat16>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_matmul_kernel<XNQ_Q4_1>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_matmul_kernel<XNQ_Q5_0>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_matmul_kernel<XNQ_Q5_1>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_matmul_kernel<XNQ_Q2K>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_matmul_kernel<XNQ_Q3K>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, generic_matmul_kernel<XNQ_Q5K>));
  return XNQ_OK;
}

} // namespace xnq
