// GGUF <-> device layout conversion, full-tensor dequantize, bias add.
//
// None of this is on the decode hot path: relayout runs once per weight at upload, dequantize is
// the API's counterpart of Q8Tensor::dequantize (xn-core/src/cuda_backend/q8.rs:94-113). What
// matters here is exactness: dequantize is bit-identical to GgmlType::to_float, so every float
// operation is an explicit round-to-nearest intrinsic the compiler may not contract into an FMA.
#include <algorithm>

#include "xnq_common.cuh"
#include "xnq_unpack.cuh"

namespace xnq {

namespace {

constexpr int TPB = 256;

// ---- GGUF blocks -> device layout, one thread per block ------------------------------------------
__global__ void relayout_q4_0(const uint8_t *__restrict__ src, uint8_t *__restrict__ qs, __half *__restrict__ d,
                              int64_t n, int64_t nblk, int64_t dstride) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n * nblk) return;
  const int64_t row = i / nblk, b = i % nblk;
  const uint16_t *s = reinterpret_cast<const uint16_t *>(src + i * 18); // blocks are 2-byte aligned
  reinterpret_cast<uint16_t *>(d)[row * dstride + b] = s[0];
  uint16_t *o = reinterpret_cast<uint16_t *>(qs + i * 16);
#pragma unroll
  for (int j = 0; j < 8; j++) o[j] = s[1 + j];
}

__global__ void relayout_q8_0(const uint8_t *__restrict__ src, uint8_t *__restrict__ qs, __half *__restrict__ d,
                              int64_t n, int64_t nblk, int64_t dstride) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n * nblk) return;
  const int64_t row = i / nblk, b = i % nblk;
  const uint16_t *s = reinterpret_cast<const uint16_t *>(src + i * 34);
  reinterpret_cast<uint16_t *>(d)[row * dstride + b] = s[0];
  uint16_t *o = reinterpret_cast<uint16_t *>(qs + i * 32);
#pragma unroll
  for (int j = 0; j < 16; j++) o[j] = s[1 + j];
}

// one thread per 2 bytes of a 210-byte super-block (105 threads of work per block)
__global__ void relayout_q6k(const uint8_t *__restrict__ src, uint8_t *__restrict__ ql, uint8_t *__restrict__ qh,
                             int8_t *__restrict__ sc, __half *__restrict__ d, int64_t n, int64_t nsb, int64_t dstride) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= n * nsb * 105) return;
  const int64_t blk = t / 105;
  const int w = (int)(t % 105); // 16-bit word index inside the block
  const uint16_t v = reinterpret_cast<const uint16_t *>(src + blk * 210)[w];
  if (w < 64) {
    reinterpret_cast<uint16_t *>(ql + blk * 128)[w] = v;
  } else if (w < 96) {
    reinterpret_cast<uint16_t *>(qh + blk * 64)[w - 64] = v;
  } else if (w < 104) {
    reinterpret_cast<uint16_t *>(sc + blk * 16)[w - 96] = v;
  } else {
    const int64_t row = blk / nsb, b = blk % nsb;
    reinterpret_cast<uint16_t *>(d)[row * dstride + b] = v;
  }
}

// Q4_K: blocks stay where they are; one thread per super-block re-packs the 12 scale bytes
template <bool TO_DEVICE>
__global__ void repack_q4k(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int64_t nblocks) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= nblocks) return;
  const uint4 *s = reinterpret_cast<const uint4 *>(src + i * 144);
  uint4 *o = reinterpret_cast<uint4 *>(dst + i * 144);
  uint4 hdr = s[0];
  const uint32_t in[3] = {hdr.y, hdr.z, hdr.w};
  uint32_t out[3];
  if (TO_DEVICE) k4_fields_from_gguf(in, out);
  else k4_fields_to_gguf(in, out);
  hdr.y = out[0];
  hdr.z = out[1];
  hdr.w = out[2];
  o[0] = hdr;
#pragma unroll
  for (int j = 1; j < 9; j++) o[j] = s[j];
}

// ---- device layout -> GGUF blocks ----------------------------------------------------------------
__global__ void canonical_q4_0(uint8_t *__restrict__ dst, const uint8_t *__restrict__ qs, const __half *__restrict__ d,
                               int64_t n, int64_t nblk, int64_t dstride) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n * nblk) return;
  const int64_t row = i / nblk, b = i % nblk;
  uint16_t *o = reinterpret_cast<uint16_t *>(dst + i * 18);
  o[0] = reinterpret_cast<const uint16_t *>(d)[row * dstride + b];
  const uint16_t *s = reinterpret_cast<const uint16_t *>(qs + i * 16);
#pragma unroll
  for (int j = 0; j < 8; j++) o[1 + j] = s[j];
}

__global__ void canonical_q8_0(uint8_t *__restrict__ dst, const uint8_t *__restrict__ qs, const __half *__restrict__ d,
                               int64_t n, int64_t nblk, int64_t dstride) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n * nblk) return;
  const int64_t row = i / nblk, b = i % nblk;
  uint16_t *o = reinterpret_cast<uint16_t *>(dst + i * 34);
  o[0] = reinterpret_cast<const uint16_t *>(d)[row * dstride + b];
  const uint16_t *s = reinterpret_cast<const uint16_t *>(qs + i * 32);
#pragma unroll
  for (int j = 0; j < 16; j++) o[1 + j] = s[j];
}

__global__ void canonical_q6k(uint8_t *__restrict__ dst, const uint8_t *__restrict__ ql, const uint8_t *__restrict__ qh,
                              const int8_t *__restrict__ sc, const __half *__restrict__ d, int64_t n, int64_t nsb,
                              int64_t dstride) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= n * nsb * 105) return;
  const int64_t blk = t / 105;
  const int w = (int)(t % 105);
  uint16_t v;
  if (w < 64) {
    v = reinterpret_cast<const uint16_t *>(ql + blk * 128)[w];
  } else if (w < 96) {
    v = reinterpret_cast<const uint16_t *>(qh + blk * 64)[w - 64];
  } else if (w < 104) {
    v = reinterpret_cast<const uint16_t *>(sc + blk * 16)[w - 96];
  } else {
    const int64_t row = blk / nsb, b = blk % nsb;
    v = reinterpret_cast<const uint16_t *>(d)[row * dstride + b];
  }
  reinterpret_cast<uint16_t *>(dst + blk * 210)[w] = v;
}

// ---- dequantize: one thread per element, exact to_float arithmetic --------------------------------
template <typename T>
__device__ __forceinline__ T cast_out(float v);
template <>
__device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void dequantize_kernel(WeightView w, T *__restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= w.n * w.k) return;
  const int64_t row = i / w.k;
  const int col = (int)(i % w.k);
  float v;
  switch (w.dtype) {
    case XNQ_Q4_0: v = deq_q4_0(w, row, col); break;
    case XNQ_Q8_0: v = deq_q8_0(w, row, col); break;
    case XNQ_Q4K: v = deq_q4k(w, row, col); break;
    default: v = deq_q6k(w, row, col); break;
  }
  out[i] = cast_out<T>(v);
}

__global__ void max_abs_kernel(WeightView w, unsigned int *out) {
  float m = 0.f;
  const int64_t total = w.n * w.k;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / w.k;
    const int col = (int)(i % w.k);
    float v;
    switch (w.dtype) {
      case XNQ_Q4_0: v = deq_q4_0(w, row, col); break;
      case XNQ_Q8_0: v = deq_q8_0(w, row, col); break;
      case XNQ_Q4K: v = deq_q4k(w, row, col); break;
      default: v = deq_q6k(w, row, col); break;
    }
    v = fabsf(v);
    if (v < 3.0e38f) m = fmaxf(m, v); // ignore inf / nan scales
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m)); // non-negative floats order like their bit patterns
}

__global__ void add_bias_kernel(float *__restrict__ y, const float *__restrict__ bias, int64_t m, int64_t n, int64_t ldy) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= m * n) return;
  const int64_t r = i / n, c = i % n;
  y[r * ldy + c] = __fadd_rn(y[r * ldy + c], bias[c]);
}

inline unsigned grid_for(int64_t work) { return (unsigned)((work + TPB - 1) / TPB); }

} // namespace

int launch_relayout(const WeightView &v, const uint8_t *src, cudaStream_t s) {
  if (v.n == 0) return XNQ_OK;
  const int64_t nblk = v.k / block_size(v.dtype);
  switch (v.dtype) {
    case XNQ_Q4_0:
      relayout_q4_0<<<grid_for(v.n * nblk), TPB, 0, s>>>(src, const_cast<uint8_t *>(v.qs), const_cast<__half *>(v.d), v.n, nblk, v.dstride);
      break;
    case XNQ_Q8_0:
      relayout_q8_0<<<grid_for(v.n * nblk), TPB, 0, s>>>(src, const_cast<uint8_t *>(v.qs), const_cast<__half *>(v.d), v.n, nblk, v.dstride);
      break;
    case XNQ_Q6K:
      relayout_q6k<<<grid_for(v.n * nblk * 105), TPB, 0, s>>>(src, const_cast<uint8_t *>(v.qs), const_cast<uint8_t *>(v.qh),
                                                              const_cast<int8_t *>(v.sc), const_cast<__half *>(v.d), v.n, nblk, v.dstride);
      break;
    case XNQ_Q4K: repack_q4k<true><<<grid_for(v.n * nblk), TPB, 0, s>>>(src, const_cast<uint8_t *>(v.qs), v.n * nblk); break;
    default: return fail(XNQ_ERR_DTYPE, "relayout: dtype %d", v.dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int launch_to_canonical(const WeightView &v, uint8_t *dst, cudaStream_t s) {
  if (v.n == 0) return XNQ_OK;
  const int64_t nblk = v.k / block_size(v.dtype);
  switch (v.dtype) {
    case XNQ_Q4_0: canonical_q4_0<<<grid_for(v.n * nblk), TPB, 0, s>>>(dst, v.qs, v.d, v.n, nblk, v.dstride); break;
    case XNQ_Q8_0: canonical_q8_0<<<grid_for(v.n * nblk), TPB, 0, s>>>(dst, v.qs, v.d, v.n, nblk, v.dstride); break;
    case XNQ_Q6K: canonical_q6k<<<grid_for(v.n * nblk * 105), TPB, 0, s>>>(dst, v.qs, v.qh, v.sc, v.d, v.n, nblk, v.dstride); break;
    case XNQ_Q4K: repack_q4k<false><<<grid_for(v.n * nblk), TPB, 0, s>>>(v.qs, dst, v.n * nblk); break;
    default: return fail(XNQ_ERR_DTYPE, "to_canonical: dtype %d", v.dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int launch_dequantize(const WeightView &w, int out_dtype, void *dst, cudaStream_t s) {
  if (w.n == 0) return XNQ_OK;
  const unsigned g = grid_for(w.n * w.k);
  switch (out_dtype) {
    case XNQ_F32: dequantize_kernel<float><<<g, TPB, 0, s>>>(w, static_cast<float *>(dst)); break;
    case XNQ_F16: dequantize_kernel<__half><<<g, TPB, 0, s>>>(w, static_cast<__half *>(dst)); break;
    case XNQ_BF16: dequantize_kernel<__nv_bfloat16><<<g, TPB, 0, s>>>(w, static_cast<__nv_bfloat16 *>(dst)); break;
    default: return fail(XNQ_ERR_DTYPE, "dequantize: output dtype %d is not f32/f16/bf16", out_dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int launch_max_abs(const WeightView &w, float *dev_out, cudaStream_t s) {
  XNQ_CUDA(cudaMemsetAsync(dev_out, 0, sizeof(float), s));
  if (w.n == 0) return XNQ_OK;
  const int64_t total = w.n * w.k;
  const unsigned grid = (unsigned)std::min<int64_t>((total + TPB - 1) / TPB, 148 * 16);
  max_abs_kernel<<<grid, TPB, 0, s>>>(w, reinterpret_cast<unsigned int *>(dev_out));
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int launch_add_bias(float *y, const float *bias, int64_t m, int64_t n, int64_t ldy, cudaStream_t s) {
  if (m == 0 || n == 0) return XNQ_OK;
  add_bias_kernel<<<grid_for(m * n), TPB, 0, s>>>(y, bias, m, n, ldy);
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int layout_init(int) {
  cudaFuncAttributes fa;
  XNQ_CUDA(cudaFuncGetAttributes(&fa, relayout_q4_0));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, relayout_q8_0));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, relayout_q6k));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, canonical_q4_0));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, canonical_q8_0));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, canonical_q6k));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, repack_q4k<true>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, repack_q4k<false>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, dequantize_kernel<float>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, dequantize_kernel<__half>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, dequantize_kernel<__nv_bfloat16>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, add_bias_kernel));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, max_abs_kernel));
  return XNQ_OK;
}

} // namespace xnq
