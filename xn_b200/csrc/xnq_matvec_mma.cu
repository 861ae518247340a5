// Small-batch decode (5 <= m <= 16) for Q4_K weights on the integer tensor-core instruction
// mma.sync.m16n8k32 (s8 x s8 -> s32).
//
// The reference's dots are exact integer sums over one 32-element sub-block, scaled in f32
// (k_quants.rs:1337-1416). A k = 32 integer MMA computes exactly those sums for 16 weight rows x 8
// activation rows at once, so the arithmetic is unchanged (the same integers, the same f32 scaling per
// sub-block) while the instruction count per weight byte drops by more than an order of magnitude against
// one dp4a per four products. On this part the instruction runs at about 30 T multiply-adds per second, the
// rate dp4a reaches only on paper, which makes a batch of 16 twice as fast as the dp4a kernel (32 us
// against 64 us on 14336 x 4096); below five rows, and for Q8_0 (whose per-block f32 scaling costs as much
// as the dots), the dp4a kernels are as fast or faster and keep the job.
//
// One warp owns 16 weight rows for the whole of k. Per 256-element super-block a lane reads, for its two
// rows (g and g + 8, g = lane / 4), eight bytes of every 32-byte chunk: lane t = lane % 4 takes bytes
// 8t..8t+7, so the four lanes of a row read one full 32-byte sector. The MMA's k index is a free
// permutation as long as both operands agree: k slots 4t..4t+3 and 16+4t..16+4t+3 are given to elements
// 8t..8t+3 and 8t+4..8t+7 of the sub-block, which makes a lane's activation fragment eight consecutive
// bytes of the activation row as well. The quantized activations are staged once per CTA in that
// fragment order (padded to 80 bytes per lane: conflict-free 8-byte reads), together with the
// per-sub-block code sums and block scales the epilogue of a super-block needs.
#include <algorithm>

#include "xnq_common.cuh"
#include "xnq_unpack.cuh"

namespace xnq {
namespace {

int g_mma_sms = 148;
constexpr int WARPS = 8, THREADS = WARPS * 32;
constexpr size_t MMA_SMEM_LIMIT = 200 * 1024;
constexpr int LANE_WORDS = 20; // 16 words of fragments per lane and super-block, padded to an odd multiple of 16 bytes

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint2 ldg8(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void store_y(void *y, int y_dtype, int64_t idx, float v) {
  if (y_dtype == XNQ_F32) static_cast<float *>(y)[idx] = v;
  else if (y_dtype == XNQ_F16) static_cast<__half *>(y)[idx] = __float2half_rn(v);
  else static_cast<__nv_bfloat16 *>(y)[idx] = __float2bfloat16_rn(v);
}

// Shared-memory image of the activations, per 256-element span s and group nb of 8 activation rows:
//   frag [s][nb][lane][LANE_WORDS]  lane (g, t): words 2j, 2j+1 = bytes 8t..8t+7 of 32-element block j of row nb*8+g
//   bsum [s][nb][t][8 j][2]         int16: sum of the 32 codes of block j for rows nb*8 + 2t, 2t+1
//   dact [s][nb][t][DPS][2]         f32 activation block scales of rows nb*8 + 2t, 2t+1 (DPS scales per span: 1 for Q8_K)
template <int NB, int DPS>
struct Stage {
  uint32_t *frag;
  int16_t *bsum;
  float *dact;
  __device__ __forceinline__ Stage(unsigned char *smem, int nspan) {
    frag = reinterpret_cast<uint32_t *>(smem);
    bsum = reinterpret_cast<int16_t *>(smem + (size_t)nspan * NB * 32 * LANE_WORDS * 4);
    dact = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(bsum) + (size_t)nspan * NB * 4 * 16 * 2);
  }
};
template <int NB, int DPS>
__host__ __device__ constexpr size_t stage_bytes(int64_t nspan) {
  return (size_t)nspan * NB * (32 * LANE_WORDS * 4 + 4 * 16 * 2 + 4 * DPS * 2 * 4);
}

template <int NB, int DPS>
__device__ __forceinline__ void stage_acts(const Stage<NB, DPS> &st, const ActView &a, int span0, int nspan) {
  const int64_t k = a.k;
  const int m = (int)a.m;
  // fragments: thread -> (s, nb, g, j, t); (j, t) walk 256 consecutive bytes of one activation row
  for (int i = threadIdx.x; i < nspan * NB * 8 * 32; i += blockDim.x) {
    const int t = i & 3, j = (i >> 2) & 7, g = (i >> 5) & 7, nb = (i >> 8) % NB, s = (i >> 8) / NB;
    const int row = nb * 8 + g;
    uint2 v = make_uint2(0, 0);
    if (row < m) v = *reinterpret_cast<const uint2 *>(a.q + (int64_t)row * k + (span0 + s) * 256 + j * 32 + t * 8);
    *reinterpret_cast<uint2 *>(st.frag + ((size_t)(s * NB + nb) * 32 + g * 4 + t) * LANE_WORDS + 2 * j) = v;
  }
  for (int i = threadIdx.x; i < nspan * NB * 4 * 8 * 2; i += blockDim.x) {
    const int e = i & 1, j = (i >> 1) & 7, t = (i >> 4) & 3, nb = (i >> 6) % NB, s = (i >> 6) / NB;
    const int row = nb * 8 + 2 * t + e;
    int v = 0;
    if (row < m) {
      const int16_t *b = a.bsum + (int64_t)row * (k / 16) + (span0 + s) * 16 + 2 * j;
      v = (int)b[0] + (int)b[1];
    }
    st.bsum[i] = (int16_t)v;
  }
  for (int i = threadIdx.x; i < nspan * NB * 4 * DPS * 2; i += blockDim.x) {
    const int e = i & 1, dj = (i >> 1) % DPS, t = ((i >> 1) / DPS) & 3, nb = ((i >> 1) / DPS / 4) % NB, s = ((i >> 1) / DPS / 4) / NB;
    const int row = nb * 8 + 2 * t + e;
    st.dact[i] = row < m ? a.d[(int64_t)row * (k / 256) * DPS + (span0 + s) * DPS + dj] : 0.f;
  }
  __syncthreads();
}

// The ks warps of a row group add their partial sums in a fixed order (k-part 0 first) and part 0 stores.
template <int NB>
__device__ __forceinline__ void reduce_and_store(float (&acc)[NB][4], float *red, int ks, int warp, int lane, bool live, int m, int64_t r0, int64_t r1,
                                                 int64_t n, void *y, int y_dtype, int64_t ldy, bool accumulate) {
  const int t = lane & 3;
  if (ks > 1) {
    __syncthreads(); // the previous round's partials have been read
#pragma unroll
    for (int nb = 0; nb < NB; nb++)
#pragma unroll
      for (int v = 0; v < 4; v++) red[(warp * NB * 4 + nb * 4 + v) * 32 + lane] = acc[nb][v];
    __syncthreads();
    if (warp % ks != 0) return;
    for (int p = 1; p < ks; p++)
#pragma unroll
      for (int nb = 0; nb < NB; nb++)
#pragma unroll
        for (int v = 0; v < 4; v++) acc[nb][v] += red[((warp + p) * NB * 4 + nb * 4 + v) * 32 + lane];
  }
  if (!live) return;
#pragma unroll
  for (int nb = 0; nb < NB; nb++)
#pragma unroll
    for (int v = 0; v < 4; v++) {
      const int act = nb * 8 + 2 * t + (v & 1);
      const int64_t row = (v & 2) ? r1 : r0;
      if (act < m && row < n) {
        if (accumulate) atomicAdd(static_cast<float *>(y) + (int64_t)act * ldy + row, acc[nb][v]); // two summands per output: order-free
        else store_y(y, y_dtype, (int64_t)act * ldy + row, acc[nb][v]);
      }
    }
}

// ---- Q4_K ----------------------------------------------------------------------------------------------
template <int NB>
__global__ void __launch_bounds__(THREADS, 2) matvec_mma_q4k(WeightView w, ActView a, void *y, int y_dtype, int64_t ldy, int ks, int nkp) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int nsb = (int)(w.k / QK_K);
  // With nkp > 1 a CTA stages and works on one of nkp runs of super-blocks only (the whole activation image
  // of a large k does not fit shared memory) and the runs' results meet in y by atomic adds: y starts at zero.
  const int kp = blockIdx.x % nkp;
  const int sp0 = nsb * kp / nkp, spn = nsb * (kp + 1) / nkp - sp0;
  const Stage<NB, 1> st(smem, spn);
  stage_acts<NB, 1>(st, a, sp0, spn);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int m = (int)a.m;
  const int64_t ngroups = (w.n + 15) / 16;
  // ks warps share a group of 16 rows and split its super-blocks, so that enough loads are in flight even
  // when n / 16 is small against the number of warps the machine holds
  const int rgl = warp / ks, kpart = warp % ks, RG = WARPS / ks;
  const int sb0 = spn * kpart / ks, sb1 = spn * (kpart + 1) / ks; // relative to this CTA's run
  float *red = reinterpret_cast<float *>(smem + stage_bytes<NB, 1>(spn)); // [WARPS][NB * 4][32]
  for (int64_t cg = blockIdx.x / nkp; cg * RG < ngroups; cg += gridDim.x / nkp) {
    const int64_t rg = cg * RG + rgl;
    const bool live = rg < ngroups;
    const int64_t r0 = rg * 16 + g, r1 = r0 + 8;
    const uint8_t *p0 = w.qs + ((r0 < w.n ? r0 : w.n - 1) * nsb + sp0 + sb0) * 144; // rows past the end read a valid row and are never stored
    const uint8_t *p1 = w.qs + ((r1 < w.n ? r1 : w.n - 1) * nsb + sp0 + sb0) * 144;
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; nb++)
#pragma unroll
      for (int v = 0; v < 4; v++) acc[nb][v] = 0.f;
    // software pipeline: the next super-block's bytes are requested before this one's are used
    uint4 h0 = ldg16(p0), h1 = ldg16(p1);
    uint2 q0[4], q1[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
      q0[c] = ldg8(p0 + 16 + 32 * c + 8 * t);
      q1[c] = ldg8(p1 + 16 + 32 * c + 8 * t);
    }
    for (int s = sb0; s < sb1 && live; s++) {
      const uint4 ch0 = h0, ch1 = h1;
      uint2 cq0[4], cq1[4];
#pragma unroll
      for (int c = 0; c < 4; c++) cq0[c] = q0[c], cq1[c] = q1[c];
      if (s + 1 < sb1) {
        const int o = (s + 1 - sb0) * 144;
        h0 = ldg16(p0 + o);
        h1 = ldg16(p1 + o);
#pragma unroll
        for (int c = 0; c < 4; c++) {
          q0[c] = ldg8(p0 + o + 16 + 32 * c + 8 * t);
          q1[c] = ldg8(p1 + o + 16 + 32 * c + 8 * t);
        }
      }
      int t1[NB][4], t2[NB][4];
#pragma unroll
      for (int nb = 0; nb < NB; nb++)
#pragma unroll
        for (int v = 0; v < 4; v++) t1[nb][v] = t2[nb][v] = 0;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const uint32_t f0 = k4_field(ch0.y, ch0.z, ch0.w, c), f1 = k4_field(ch1.y, ch1.z, ch1.w, c);
        const int sc0[2] = {(int)(f0 & 63), (int)((f0 >> 6) & 63)}, mn0[2] = {(int)((f0 >> 12) & 63), (int)(f0 >> 18)};
        const int sc1[2] = {(int)(f1 & 63), (int)((f1 >> 6) & 63)}, mn1[2] = {(int)((f1 >> 12) & 63), (int)(f1 >> 18)};
#pragma unroll
        for (int hl = 0; hl < 2; hl++) { // sub-block 2c (low nibbles), 2c + 1 (high nibbles)
          const int j = 2 * c + hl;
          const uint32_t a0 = (cq0[c].x >> (4 * hl)) & 0x0f0f0f0fu, a1 = (cq1[c].x >> (4 * hl)) & 0x0f0f0f0fu;
          const uint32_t a2 = (cq0[c].y >> (4 * hl)) & 0x0f0f0f0fu, a3 = (cq1[c].y >> (4 * hl)) & 0x0f0f0f0fu;
#pragma unroll
          for (int nb = 0; nb < NB; nb++) {
            const uint2 b = *reinterpret_cast<const uint2 *>(st.frag + ((size_t)(s * NB + nb) * 32 + lane) * LANE_WORDS + 2 * j);
            int cc[4] = {0, 0, 0, 0};
            mma_s8(cc, a0, a1, a2, a3, b.x, b.y);
            const uint32_t bs = *reinterpret_cast<const uint32_t *>(st.bsum + (((size_t)(s * NB + nb) * 4 + t) * 8 + j) * 2);
            const int bs_e0 = (int)(int16_t)(bs & 0xffff), bs_e1 = (int)(int16_t)(bs >> 16);
            t1[nb][0] += sc0[hl] * cc[0], t1[nb][1] += sc0[hl] * cc[1], t1[nb][2] += sc1[hl] * cc[2], t1[nb][3] += sc1[hl] * cc[3];
            t2[nb][0] += mn0[hl] * bs_e0, t2[nb][1] += mn0[hl] * bs_e1, t2[nb][2] += mn1[hl] * bs_e0, t2[nb][3] += mn1[hl] * bs_e1;
          }
        }
      }
      const __half2 dm0 = *reinterpret_cast<const __half2 *>(&ch0.x), dm1 = *reinterpret_cast<const __half2 *>(&ch1.x);
      const float d0 = __low2float(dm0), m0 = __high2float(dm0), d1 = __low2float(dm1), m1 = __high2float(dm1);
#pragma unroll
      for (int nb = 0; nb < NB; nb++) {
        const float2 da = *reinterpret_cast<const float2 *>(st.dact + ((size_t)(s * NB + nb) * 4 + t) * 2);
        acc[nb][0] += da.x * (d0 * (float)t1[nb][0] - m0 * (float)t2[nb][0]);
        acc[nb][1] += da.y * (d0 * (float)t1[nb][1] - m0 * (float)t2[nb][1]);
        acc[nb][2] += da.x * (d1 * (float)t1[nb][2] - m1 * (float)t2[nb][2]);
        acc[nb][3] += da.y * (d1 * (float)t1[nb][3] - m1 * (float)t2[nb][3]);
      }
    }
    reduce_and_store<NB>(acc, red, ks, warp, lane, live, m, r0, r1, w.n, y, y_dtype, ldy, nkp > 1);
  }
}

constexpr size_t RED_BYTES = (size_t)WARPS * 2 * 4 * 32 * 4; // the k-split partials of a CTA

template <int NB>
int launch_nb(const WeightView &w, const ActView &a, void *y, int y_dtype, int64_t ldy, cudaStream_t s) {
  const int64_t nspan = w.k / 256;
  // the activation image of the whole k, or of one of two halves of it when that is what fits
  int nkp = 1;
  if (stage_bytes<NB, 1>(nspan) + RED_BYTES > MMA_SMEM_LIMIT) nkp = 2;
  const int64_t spn = (nspan + nkp - 1) / nkp;
  const size_t sm = stage_bytes<NB, 1>(spn) + RED_BYTES;
  if (sm > MMA_SMEM_LIMIT || (nkp > 1 && y_dtype != XNQ_F32)) return fail(XNQ_ERR_SIZE, "matvec_mma: k = %lld does not fit", (long long)w.k);
  const int per_sm = sm > 110 * 1024 ? 1 : 2;
  // split k over as many warps as it takes to fill the machine (depends on the weight's shape only, so the
  // summation order of a row is the same for every batch size)
  const int64_t ngroups = (w.n + 15) / 16, slots = (int64_t)g_mma_sms * 2 * WARPS;
  int ks = 1;
  while (ks < WARPS && ngroups * ks * nkp < slots && spn / (ks * 2) >= 2) ks *= 2;
  const int64_t cta_groups = (ngroups + WARPS / ks - 1) / (WARPS / ks);
  const unsigned grid = (unsigned)(std::max<int64_t>(1, std::min<int64_t>(cta_groups, (int64_t)g_mma_sms * per_sm / nkp)) * nkp);
  if (nkp > 1) XNQ_CUDA(cudaMemset2DAsync(y, (size_t)ldy * 4, 0, (size_t)w.n * 4, (size_t)a.m, s)); // the halves add into zeros
  matvec_mma_q4k<NB><<<grid, THREADS, sm, s>>>(w, a, y, y_dtype, ldy, ks, nkp);
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

} // namespace

// Activation rows one launch can stage for this weight (0: this kernel does not serve it).
int64_t matvec_mma_rows_per_pass(const WeightView &w, int y_dtype) {
  if (w.dtype != XNQ_Q4K || w.n < 1) return 0;
  const int64_t nspan = w.k / 256;
  if (stage_bytes<2, 1>(nspan) + RED_BYTES <= MMA_SMEM_LIMIT) return 16;
  if (y_dtype == XNQ_F32 && stage_bytes<2, 1>((nspan + 1) / 2) + RED_BYTES <= MMA_SMEM_LIMIT) return 16; // two half-k images, summed in y
  if (stage_bytes<1, 1>(nspan) + RED_BYTES <= MMA_SMEM_LIMIT) return 8;
  return 0;
}

// Whether a launch for m rows splits k between CTAs that add into a zeroed y with atomics (y must then be
// ordinary device memory: atomics on mapped host memory are not atomic for the host and cross the host link one by one).
bool matvec_mma_accumulates_in_y(const WeightView &w, int64_t m) {
  if (w.dtype != XNQ_Q4K) return false;
  const int64_t nspan = w.k / 256;
  return (m <= 8 ? stage_bytes<1, 1>(nspan) : stage_bytes<2, 1>(nspan)) + RED_BYTES > MMA_SMEM_LIMIT;
}

int launch_matvec_mma(const WeightView &w, const ActView &a, void *y, int y_dtype, int64_t ldy, cudaStream_t s) {
  if (w.n == 0 || a.m == 0) return XNQ_OK;
  const int64_t pass = matvec_mma_rows_per_pass(w, y_dtype);
  if (a.m > pass) return fail(XNQ_ERR_SHAPE, "matvec_mma: m = %lld exceeds the %lld rows one launch stages", (long long)a.m, (long long)pass);
  return a.m <= 8 ? launch_nb<1>(w, a, y, y_dtype, ldy, s) : launch_nb<2>(w, a, y, y_dtype, ldy, s);
}

int matvec_mma_init(int device) {
  cudaDeviceProp prop;
  XNQ_CUDA(cudaGetDeviceProperties(&prop, device));
  g_mma_sms = prop.multiProcessorCount;
  XNQ_CUDA(cudaFuncSetAttribute(matvec_mma_q4k<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_LIMIT));
  XNQ_CUDA(cudaFuncSetAttribute(matvec_mma_q4k<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_LIMIT));
  return XNQ_OK;
}

} // namespace xnq
