// Activation quantizers: f32 / f16 / bf16 rows -> Q8_0 or Q8_K blocks, bit-exact with the CPU path.
//
//   Q8_0 (for Q4_0 / Q8_0 weights): BlockQ8_0::from_float, xn-core/src/quantized/k_quants.rs:636-661
//   Q8_K (for Q4_K / Q6_K weights): BlockQ8K::from_float,  k_quants.rs:1942-1979
//
// Each thread owns 8 consecutive elements; a Q8_0 block is 4 lanes, a Q8_K block one whole warp.
// Output is either the canonical block bytes (the parity-tested public entry) or the planar scratch
// the matmul kernels read. Both come from the same arithmetic, shared through quantize_act.cuh.
#include "xnq_common.cuh"
#include "xnq_quantize_act.cuh"

namespace xnq {

size_t act_workspace_bytes(int64_t m, int64_t k, int act_dtype) {
  const int64_t blk = act_dtype == XNQ_Q8_0 ? QK : QK_K;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  return up((size_t)m * k) + up((size_t)m * (k / blk) * 4) + up((size_t)m * (k / 16) * 2);
}

ActView act_view(void *ws, int64_t m, int64_t k, int act_dtype) {
  const int64_t blk = act_dtype == XNQ_Q8_0 ? QK : QK_K;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  ActView a;
  a.act_dtype = act_dtype;
  a.m = m;
  a.k = k;
  char *p = static_cast<char *>(ws);
  a.q = reinterpret_cast<int8_t *>(p);
  p += up((size_t)m * k);
  a.d = reinterpret_cast<float *>(p);
  p += up((size_t)m * (k / blk) * 4);
  a.bsum = reinterpret_cast<int16_t *>(p);
  return a;
}

namespace {

constexpr int TPB = 256;

// LAYOUT 0: canonical GGUF activation blocks; LAYOUT 1: planar scratch
template <int ACT, typename XT, int LAYOUT>
__global__ void __launch_bounds__(TPB) quantize_act_kernel(const XT *__restrict__ x, int64_t m, int64_t k, int64_t ldx,
                                                           uint8_t *__restrict__ blocks, ActView pl) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t per_row = k / 8;
  const bool valid = t < m * per_row;
  const int64_t row = valid ? t / per_row : 0;
  const int64_t c8 = valid ? t % per_row : 0;
  float v[8];
  if (valid) {
    load8(x + row * ldx + c8 * 8, v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = 0.f;
  }
  const int lane = threadIdx.x & 31;
  Quant8 q = ACT == XNQ_Q8_0 ? quantize8_q8_0(v, lane) : quantize8_q8k(v, lane);
  if (!valid) return;

  if (LAYOUT == 1) {
    *reinterpret_cast<uint2 *>(pl.q + row * k + c8 * 8) = make_uint2(q.lo, q.hi);
    if (ACT == XNQ_Q8_0) {
      if ((lane & 3) == 0) pl.d[row * (k / QK) + c8 / 4] = q.d;
    } else {
      if (lane == 0) pl.d[row * (k / QK_K) + c8 / 32] = q.d;
    }
    if ((lane & 1) == 0) pl.bsum[row * (k / 16) + c8 / 2] = (int16_t)q.sum16;
  } else if (ACT == XNQ_Q8_0) {
    uint8_t *b = blocks + (row * (k / QK) + c8 / 4) * 34; // 2-byte aligned
    if ((lane & 3) == 0) *reinterpret_cast<__half *>(b) = __float2half_rn(q.d_unrounded);
    uint16_t *o = reinterpret_cast<uint16_t *>(b + 2 + 8 * (c8 & 3));
    o[0] = (uint16_t)(q.lo & 0xffff);
    o[1] = (uint16_t)(q.lo >> 16);
    o[2] = (uint16_t)(q.hi & 0xffff);
    o[3] = (uint16_t)(q.hi >> 16);
  } else {
    uint8_t *b = blocks + (row * (k / QK_K) + c8 / 32) * 292; // 4-byte aligned
    if (lane == 0) *reinterpret_cast<float *>(b) = q.d;
    uint32_t *o = reinterpret_cast<uint32_t *>(b + 4 + 8 * (c8 & 31));
    o[0] = q.lo;
    o[1] = q.hi;
    if ((lane & 1) == 0) *reinterpret_cast<int16_t *>(b + 260 + 2 * ((c8 & 31) / 2)) = (int16_t)q.sum16;
  }
}

template <int ACT, int LAYOUT>
int launch_typed(const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx, uint8_t *blocks, const ActView &pl, cudaStream_t s) {
  const int64_t threads = m * (k / 8);
  if (threads == 0) return XNQ_OK;
  const unsigned grid = (unsigned)((threads + TPB - 1) / TPB);
  switch (x_dtype) {
    case XNQ_F32: quantize_act_kernel<ACT, float, LAYOUT><<<grid, TPB, 0, s>>>(static_cast<const float *>(x), m, k, ldx, blocks, pl); break;
    case XNQ_F16: quantize_act_kernel<ACT, __half, LAYOUT><<<grid, TPB, 0, s>>>(static_cast<const __half *>(x), m, k, ldx, blocks, pl); break;
    case XNQ_BF16:
      quantize_act_kernel<ACT, __nv_bfloat16, LAYOUT><<<grid, TPB, 0, s>>>(static_cast<const __nv_bfloat16 *>(x), m, k, ldx, blocks, pl);
      break;
    default: return fail(XNQ_ERR_DTYPE, "quantize_act: activation dtype %d is not f32/f16/bf16", x_dtype);
  }
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

} // namespace

int launch_quantize_act_blocks(int act_dtype, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx, void *dst, cudaStream_t s) {
  ActView none{};
  if (act_dtype == XNQ_Q8_0) return launch_typed<XNQ_Q8_0, 0>(x, x_dtype, m, k, ldx, static_cast<uint8_t *>(dst), none, s);
  if (act_dtype == XNQ_Q8K) return launch_typed<XNQ_Q8K, 0>(x, x_dtype, m, k, ldx, static_cast<uint8_t *>(dst), none, s);
  return fail(XNQ_ERR_DTYPE, "quantize_act: %d is not an activation block format (Q8_0=8, Q8K=15)", act_dtype);
}

int launch_quantize_act_planar(const ActView &a, const void *x, int x_dtype, int64_t ldx, cudaStream_t s) {
  if (a.act_dtype == XNQ_Q8_0) return launch_typed<XNQ_Q8_0, 1>(x, x_dtype, a.m, a.k, ldx, nullptr, a, s);
  return launch_typed<XNQ_Q8K, 1>(x, x_dtype, a.m, a.k, ldx, nullptr, a, s);
}

int quantize_init(int) {
  cudaFuncAttributes fa;
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8_0, float, 0>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8_0, float, 1>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8K, float, 0>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8K, float, 1>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8_0, __half, 1>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8K, __half, 1>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8_0, __nv_bfloat16, 1>));
  XNQ_CUDA(cudaFuncGetAttributes(&fa, quantize_act_kernel<XNQ_Q8K, __nv_bfloat16, 1>));
  return XNQ_OK;
}

} // namespace xnq
