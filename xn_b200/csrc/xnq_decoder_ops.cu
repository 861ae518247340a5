// The small operators that sit between the quantized linears of a Llama-style decode step, fused so a
// step is a handful of launches per layer instead of dozens: residual-add + RMSNorm, RoPE + KV-cache
// store, single-query attention over the cache, SwiGLU. They are the callers of the quantized matmul
// path in the reference's model (xn-core/src/models/llama.rs:145-216, 258-265, 300-320) and follow
// its arithmetic: RMSNorm as x * rsqrt(mean(x^2) + eps) * w, rotate-half RoPE, softmax(q k^T / sqrt(d)) v
// with grouped-query heads, silu(gate) * up. All f32 math; the KV cache is bf16.
#include "xnq_common.cuh"
#include "xnq_quantize_act.cuh"

namespace xnq {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Planar activation image of one row (the layout of act_view): codes, block scales, 16-element sums.
struct RowImage {
  int8_t *q;
  float *d;
  int16_t *bsum;
};
__device__ __forceinline__ RowImage row_image(void *image, int64_t rows, int64_t k, int blk, int64_t row) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  char *p = static_cast<char *>(image);
  RowImage r;
  r.q = reinterpret_cast<int8_t *>(p) + row * k;
  p += up((size_t)rows * k);
  r.d = reinterpret_cast<float *>(p) + row * (k / blk);
  p += up((size_t)rows * (k / blk) * 4);
  r.bsum = reinterpret_cast<int16_t *>(p) + row * (k / 16);
  return r;
}
// Quantizes the 8 values of this lane (elements c8 * 8 .. of the row; a warp holds 256 consecutive elements)
// and stores them into the row's image. All 32 lanes call it; lanes past the end of the row pass zeros.
template <int ACT>
__device__ __forceinline__ void quantize_store8(const float (&v)[8], bool valid, const RowImage &img, int64_t c8, int lane) {
  const Quant8 q = ACT == XNQ_Q8_0 ? quantize8_q8_0(v, lane) : quantize8_q8k(v, lane);
  if (!valid) return;
  *reinterpret_cast<uint2 *>(img.q + c8 * 8) = make_uint2(q.lo, q.hi);
  if (ACT == XNQ_Q8_0) {
    if ((lane & 3) == 0) img.d[c8 / 4] = q.d;
  } else {
    if (lane == 0) img.d[c8 / 32] = q.d;
  }
  if ((lane & 1) == 0) img.bsum[c8 / 2] = (int16_t)q.sum16;
}

// The same 8 values into an OPERAND image (the integer tensor-core kernel's layout, xnq_common.cuh): k8 = index of the lane's first
// element in the row (a warp holds one 256-element block, lane = (k8 / 8) % 32).
constexpr int ACT_OPERAND = XNQ_ACT_OPERAND;
__device__ __forceinline__ void quantize_store8_operand(const float (&v)[8], bool valid, void *image, int64_t rows, int64_t k, int64_t row, int64_t k8, int lane) {
  const Quant8 q = quantize8_q8k(v, lane);
  const int sum16 = q.sum16;
  const int s32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 2); // lanes 4 s .. 4 s + 3 hold sub-block s; sum16 is a lane pair's sum on both lanes
  const int sub = lane >> 2;
  uint32_t lo_b = (lane & 3) == 0 ? ((uint32_t)(s32 & 127) << (8 * (sub & 3))) : 0u;
  uint32_t hi_b = (lane & 3) == 0 ? ((uint32_t)((s32 >> 7) & 0xff) << (8 * (sub & 3))) : 0u;
#pragma unroll
  for (int off = 4; off <= 8; off <<= 1) {
    lo_b |= __shfl_xor_sync(0xffffffffu, lo_b, off);
    hi_b |= __shfl_xor_sync(0xffffffffu, hi_b, off);
  }
  if (!valid) return;
  const int NP = operand_np(rows);
  uint8_t *bimg = static_cast<uint8_t *>(image) + OPERAND_TICKET_BYTES;
  uint8_t *meta = bimg + operand_bimg_bytes(NP, k);
  const int64_t hs = k8 >> 7;
  const int chunk = (int)((k8 & 127) >> 4);
  uint8_t *dst = bimg + (size_t)hs * (NP * 128) + (size_t)(row >> 3) * 1024 + (size_t)(row & 7) * 128 + (size_t)((chunk ^ (int)(row & 7)) << 4) + (k8 & 8);
  *reinterpret_cast<uint2 *>(dst) = make_uint2(q.lo, q.hi);
  uint32_t *rec = reinterpret_cast<uint32_t *>(meta + ((size_t)(k8 >> 8) * NP + row) * 32);
  if (lane == 0 || lane == 16) {
    rec[(lane >> 4) * 2] = lo_b;
    rec[(lane >> 4) * 2 + 1] = hi_b;
  }
  if (lane == 0) {
    rec[4] = __float_as_uint(q.d);
    rec[5] = rec[6] = rec[7] = 0u;
  }
}
// the ticket words of an OPERAND image are put back to zero by the kernel that used them; a producer zeroes them as well, so that a
// matmul that gave up half way cannot spoil the next one
__device__ __forceinline__ void operand_clear_tickets(void *image) {
  unsigned int *t = static_cast<unsigned int *>(image);
  for (int i = threadIdx.x; i < OPERAND_MAX_TILES; i += blockDim.x) t[i] = 0u;
}

// x[row] += sum_p delta[row][p] (if delta), out[row] = x[row] * rsqrt(mean(x^2) + eps) * w, and optionally the
// quantized image of out[row]. One CTA of 256 threads per row, 8 consecutive elements per thread per pass.
template <int ACT>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(float *x, const float *delta, int parts, const float *w, float eps, float *out, void *image,
                                                          int64_t rows, int d) {
  constexpr int MAXP = 128; // 256-element partial sums kept apart (rows of up to 32768 values; beyond that they wrap around)
  __shared__ float part[MAXP];
  pdl_launch_dependents();
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // The norm weights never change, and in a decode step they come from DRAM (the step's 4 GB of linear weights have been
  // through L2 since their last use): they are requested before the wait for the kernel that produces x and delta.
  constexpr int KEEP = 2;
  float kv[KEEP][8], kg[KEEP][8];
#pragma unroll
  for (int p = 0; p < KEEP; p++)
    if (p * 2048 + threadIdx.x * 8 < d) load8(w + p * 2048 + threadIdx.x * 8, kg[p]);
  pdl_wait(); // x and delta are earlier kernels' outputs
  float *xr = x + row * d;
  const float *dr = delta ? delta + row * parts * d : nullptr;
  const int np = (d + 255) / 256;
  for (int i = threadIdx.x; i < min(np, MAXP); i += 256) part[i] = 0.f;
  __syncthreads();
  // The first KEEP passes of 2048 values (rows of up to 4096 values entirely) stay in registers between the
  // sum of squares and the scaling: one trip to memory instead of three. Longer rows re-read the rest.
  // adds the summands, stores the new residual, returns the sum of squares of the thread's run of 8
  auto first_pass = [&](int i, float (&v)[8]) {
    load8(xr + i, v);
    if (dr) {
      for (int q = 0; q < parts; q++) {
        float a[8];
        load8(dr + (int64_t)q * d + i, a);
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = __fadd_rn(v[e], a[e]);
      }
      *reinterpret_cast<float4 *>(xr + i) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(xr + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    return rms_run_sum(v);
  };
  // one partial sum per 256 elements: pass p, warp w holds elements 2048 p + 256 w ..
  auto pass_sum = [&](int p, float run) {
    if (p * 2048 + warp * 256 >= d) return; // whole warps leave together
    const float s = rms_warp_sum(run);
    const int idx = p * 8 + warp;
    if (lane == 0) part[idx % MAXP] += s; // one writer per entry and pass; entries are reused only by rows longer than 32768
  };
#pragma unroll
  for (int p = 0; p < KEEP; p++) {
    const int i = p * 2048 + threadIdx.x * 8;
    float run = 0.f;
    if (i < d) run = first_pass(i, kv[p]);
    pass_sum(p, run);
  }
  for (int p = KEEP; p * 2048 < d; p++) {
    const int i = p * 2048 + threadIdx.x * 8;
    float v[8];
    pass_sum(p, i < d ? first_pass(i, v) : 0.f);
  }
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < min(np, MAXP); i++) tot += part[i];
  const float r = rms_scale(tot, d, eps);
  RowImage img{};
  if (ACT != 0 && ACT != ACT_OPERAND) img = row_image(image, rows, d, ACT == XNQ_Q8_0 ? QK : QK_K, row);
  if (ACT == ACT_OPERAND && row == 0) operand_clear_tickets(image);
  auto second_pass = [&](int base, float (&v)[8], const float (&g)[8], bool loaded) { // whole warps stay together for the quantizer's shuffles
    const int i = base + threadIdx.x * 8;
    const bool valid = i < d;
    if (valid) {
      float gg[8];
      if (!loaded) {
        load8(xr + i, v); // this thread's own stores of the first pass
        load8(w + i, gg);
      }
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] = rms_apply(v[e], r, loaded ? g[e] : gg[e]);
      if (out) {
        *reinterpret_cast<float4 *>(out + row * d + i) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(out + row * d + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] = 0.f;
    }
    if (ACT == ACT_OPERAND) quantize_store8_operand(v, valid, image, rows, d, row, i, lane);
    else if (ACT != 0) quantize_store8<ACT == ACT_OPERAND ? XNQ_Q8K : ACT>(v, valid, img, i / 8, lane);
  };
#pragma unroll
  for (int p = 0; p < KEEP; p++)
    if (p * 2048 + (threadIdx.x & ~31) * 8 < d) second_pass(p * 2048, kv[p], kg[p], true);
  for (int base = KEEP * 2048; base + (threadIdx.x & ~31) * 8 < d; base += 2048) {
    float v[8];
    second_pass(base, v, v, false);
  }
}

// out[row, j] = silu(gu[row, j]) * gu[row, f + j], optionally with its quantized image. 8 consecutive
// elements per thread; f is a multiple of 256 when an image is written, so a warp never straddles two rows.
template <int ACT>
__global__ void __launch_bounds__(256) swiglu_kernel(const float *gu, float *out, void *image, int64_t rows, int f) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t per_row = f / 8;
  const bool valid = t < rows * per_row;
  if (ACT == 0 && !valid) return;
  const int64_t r = valid ? t / per_row : 0, c8 = valid ? t - r * per_row : 0;
  float v[8];
  if (valid) {
    float g[8], u[8];
    load8(gu + r * 2 * f + c8 * 8, g);
    load8(gu + r * 2 * f + f + c8 * 8, u);
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    if (out) {
      *reinterpret_cast<float4 *>(out + r * f + c8 * 8) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(out + r * f + c8 * 8 + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = 0.f;
  }
  if (ACT == ACT_OPERAND) {
    if (blockIdx.x == 0) operand_clear_tickets(image);
    quantize_store8_operand(v, valid, image, rows, f, r, c8 * 8, threadIdx.x & 31);
  } else if (ACT != 0) {
    quantize_store8<ACT == ACT_OPERAND ? XNQ_Q8K : ACT>(v, valid, row_image(image, rows, f, ACT == XNQ_Q8_0 ? QK : QK_K, r), c8, threadIdx.x & 31);
  }
}

// x[row, :] = table[tokens[row], :] widened to f32 (bf16 table). One CTA per row, 8 elements per thread and pass. A token outside
// [0, vocab) gives a row of zeros and sets status bit 4. Launched as a plain (not programmatically dependent) kernel: it is the
// step's first kernel, and everything behind it may rely on the previous step's stores (position, tokens, cache rows) being complete.
__global__ void __launch_bounds__(256) embed_rows_kernel(const __nv_bfloat16 *table, const long long *tokens, float *x, int d, long long vocab);

// tokens[row] = index of the first largest logit of the row (torch.argmax's rule), then *pos += 1 (one thread). One CTA per row.
__global__ void __launch_bounds__(256) argmax_advance_kernel(const float *logits, long long n, long long *tokens, long long *pos);

__device__ unsigned int g_decoder_status; // sticky: 1 rope/store, 2 attention saw a position outside [0, max_seq), 4 an embedding token outside the table

__global__ void __launch_bounds__(256) embed_rows_kernel(const __nv_bfloat16 *table, const long long *tokens, float *x, int d, long long vocab) {
  const long long tok = tokens[blockIdx.x];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0) atomicOr(&g_decoder_status, 4u);
  const __nv_bfloat16 *src = table + (ok ? tok : 0) * (long long)d;
  float *dst = x + (long long)blockIdx.x * d;
  for (int i = threadIdx.x * 8; i < d; i += 256 * 8) {
    float v[8];
    if (ok) load8(src + i, v);
    else {
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] = 0.f;
    }
    *reinterpret_cast<float4 *>(dst + i) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4 *>(dst + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

__global__ void __launch_bounds__(256) argmax_advance_kernel(const float *logits, long long n, long long *tokens, long long *pos) {
  __shared__ float s_v[8];
  __shared__ long long s_i[8];
  pdl_launch_dependents();
  pdl_wait(); // the logits are the previous kernel's output
  const float *row = logits + (long long)blockIdx.x * n;
  float best = -INFINITY;
  long long bi = n; // no candidate yet
  for (long long i = threadIdx.x; i < n; i += 256) {
    const float v = row[i];
    if (v > best || (v == best && i < bi)) best = v, bi = i;
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const long long oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) s_v[warp] = best, s_i[warp] = bi;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++)
      if (s_v[w] > best || (s_v[w] == best && s_i[w] < bi)) best = s_v[w], bi = s_i[w];
    tokens[blockIdx.x] = bi < n ? bi : 0; // a row of -inf / NaN only: token 0
    if (blockIdx.x == 0 && pos) *pos += 1;
  }
}

// Rotate-half RoPE of the pair (x1 = element i, x2 = element i + hd / 2) with every operation rounded separately, so that the
// stand-alone kernel and the attention kernel that rotates in its prologue produce the same bits.
__device__ __forceinline__ float rope_lo(float x1, float x2, float c, float s) { return __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)); }
__device__ __forceinline__ float rope_hi(float x1, float x2, float c, float s) { return __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)); }

// One token per sequence. qkv [B, (H + 2 KV) * hd] f32 -> q_out [B, H, hd] f32 (rotated), and the rotated k
// and plain v of every KV head go to the caches [B, KV, max_seq, hd] (bf16) at position *pos.
// grid (H + 2 KV, B), block hd / 2.
__global__ void rope_store_kernel(const float *qkv, const float *cos_t, const float *sin_t, const long long *pos_p, float *q_out,
                                  __nv_bfloat16 *k_cache, __nv_bfloat16 *v_cache, int H, int KV, int hd, int max_seq) {
  const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = hd / 2;
  pdl_launch_dependents();
  pdl_wait();
  const long long pos = *pos_p;
  if (pos < 0 || pos >= max_seq) {
    if (head == 0 && b == 0 && i == 0) atomicOr(&g_decoder_status, 1u);
    return;
  }
  const float *src = qkv + ((int64_t)b * (H + 2 * KV) + head) * hd;
  const float x1 = src[i], x2 = src[i + half];
  if (head < H + KV) {
    const float c = cos_t[pos * half + i], s = sin_t[pos * half + i];
    const float r1 = rope_lo(x1, x2, c, s), r2 = rope_hi(x1, x2, c, s);
    if (head < H) {
      float *q = q_out + ((int64_t)b * H + head) * hd;
      q[i] = r1, q[i + half] = r2;
    } else {
      __nv_bfloat16 *k = k_cache + (((int64_t)b * KV + (head - H)) * max_seq + pos) * hd;
      k[i] = __float2bfloat16_rn(r1), k[i + half] = __float2bfloat16_rn(r2);
    }
  } else {
    __nv_bfloat16 *v = v_cache + (((int64_t)b * KV + (head - H - KV)) * max_seq + pos) * hd;
    v[i] = __float2bfloat16_rn(x1), v[i + half] = __float2bfloat16_rn(x2);
  }
}

// Single-query attention over positions 0..*pos of the cache, split over the sequence so that even one
// sequence fills the machine: grid (heads, batch, splits), 4 warps per CTA. A warp takes 32 positions
// at a time: lane j computes the whole q.k of position base + j (16 independent 16-byte loads of its
// k row), the warp turns the 32 scores into softmax weights against its running maximum, and then
// every lane accumulates its own 4 output dimensions over the 32 v rows (coalesced 256-byte rows).
// Each CTA leaves (max, sum, acc[128]) in the workspace; the last CTA of a (head, sequence) to finish
// merges the splits. The arrival counters wrap to zero by themselves (atomicInc), so the workspace
// only has to be zeroed once, when it is allocated. Workspace layout: one group per (sequence, head) pair,
// indexed b * heads + head: a 16-byte slot whose first word is the arrival counter, then ATT_MAX_SPLITS
// records. A counter's address depends on the pair's linear index alone, so a workspace may be reused by calls
// of different batch sizes and head counts (one call at a time).
// A position outside [0, max_seq) sets a sticky status bit (1 rope/store, 2 attention): the rope kernel then
// stores nothing, attention clamps a position past the cache and writes zeros for a negative one.
constexpr int ATT_WARPS = 4, ATT_HD = 128, ATT_MAX_SPLITS = 16, ATT_REC = ATT_HD + 2;
constexpr int ATT_GROUP = 4 + ATT_MAX_SPLITS * ATT_REC; // floats per (sequence, head) group

__device__ __forceinline__ void online_merge(float &m, float &l, float4 &acc, float m2, float l2, const float4 &a2) {
  const float mn = fmaxf(m, m2);
  const float f1 = m == -INFINITY ? 0.f : __expf(m - mn), f2 = m2 == -INFINITY ? 0.f : __expf(m2 - mn);
  acc = make_float4(acc.x * f1 + a2.x * f2, acc.y * f1 + a2.y * f2, acc.z * f1 + a2.z * f2, acc.w * f1 + a2.w * f2);
  l = l * f1 + l2 * f2;
  m = mn;
}

// ROPE: q is the projection output qkv [B, (H + 2 KV) * hd]; the CTA rotates its own head's q, and the CTAs whose run of positions holds the
// current one rotate that position's k (and take its v) from qkv instead of reading the cache; the first query head of every KV head also
// stores them into the caches for the steps to come. Same bits as rope_store_kernel followed by the plain kernel, one launch less.
template <bool ROPE>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_decode_kernel(const float *q, __nv_bfloat16 *k_cache, __nv_bfloat16 *v_cache, const long long *pos_p,
                                                                      float *out, float *part, int H, int KV, int max_seq, float scale, const float *cos_t,
                                                                      const float *sin_t) {
  __shared__ __align__(16) float s_q[ATT_WARPS][ATT_HD]; // every warp keeps its own copy: no block-wide barrier before the loads
  __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS];
  __shared__ __align__(16) float s_acc[ATT_WARPS][ATT_HD];
  __shared__ __align__(16) __nv_bfloat16 s_k[ATT_WARPS][32][ATT_HD + 8]; // rows padded to 272 bytes: conflict-free row reads
  __shared__ bool s_last;
  const int head = blockIdx.x, b = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = head / (H / KV);
  pdl_launch_dependents();
  // Plain form: q, the cache row of the current position and possibly the position itself are the previous kernels' outputs.
  // ROPE form: only qkv is. The position was advanced at the end of the previous decode step and the cache rows below it were
  // stored in earlier steps, both behind kernels launched without programmatic overlap (sampling, the embedding gather), which
  // complete before anything of this step starts; so the position is read and the first run of k and v rows is requested BEFORE
  // griddepcontrol.wait, under the projection kernel that is still producing qkv: the cache's trip to DRAM leaves the critical path.
  bool waited = !ROPE;
  if (!ROPE) pdl_wait();
  const long long pos = *pos_p;
  int last = (int)pos;
  if (pos < 0 || pos >= max_seq) {
    if (!waited) pdl_wait();
    waited = true;
    if (head == 0 && b == 0 && split == 0 && threadIdx.x == 0) atomicOr(&g_decoder_status, ROPE ? 3u : 2u);
    if (pos < 0) { // nothing to attend to: zeros, not 0 / 0
      if (split == 0 && threadIdx.x < ATT_HD) out[((int64_t)b * H + head) * ATT_HD + threadIdx.x] = 0.f;
      return;
    }
    last = max_seq - 1;
  }
  const int npos = last + 1, per = (npos + nsplit - 1) / nsplit;
  const int c0 = split * per, c1 = min(npos, c0 + per);
  const int fresh = ROPE && pos == last ? last : -1; // the position whose k and v are still in qkv
  const float *qsrc = ROPE ? q + ((int64_t)b * (H + 2 * KV) + head) * ATT_HD : q + ((int64_t)b * H + head) * ATT_HD;
  float4 qreg = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!ROPE) qreg = *reinterpret_cast<const float4 *>(qsrc + lane * 4); // in flight together with the first k and v loads
  float4 cs = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
  if (ROPE) { // the tables never change
    cs = *reinterpret_cast<const float4 *>(cos_t + (int64_t)last * (ATT_HD / 2) + (lane & 15) * 4);
    sn = *reinterpret_cast<const float4 *>(sin_t + (int64_t)last * (ATT_HD / 2) + (lane & 15) * 4);
  }
  auto load_rotate_q = [&]() { // lanes 0..15 hold elements i < 64, lanes 16..31 their partners i + 64
    qreg = *reinterpret_cast<const float4 *>(qsrc + lane * 4);
    float4 o;
    o.x = __shfl_xor_sync(0xffffffffu, qreg.x, 16), o.y = __shfl_xor_sync(0xffffffffu, qreg.y, 16);
    o.z = __shfl_xor_sync(0xffffffffu, qreg.z, 16), o.w = __shfl_xor_sync(0xffffffffu, qreg.w, 16);
    if (pos == last) { // a position past the cache rotates nothing, as the stand-alone kernel stores nothing
      if (lane < 16) qreg = make_float4(rope_lo(qreg.x, o.x, cs.x, sn.x), rope_lo(qreg.y, o.y, cs.y, sn.y), rope_lo(qreg.z, o.z, cs.z, sn.z), rope_lo(qreg.w, o.w, cs.w, sn.w));
      else qreg = make_float4(rope_hi(o.x, qreg.x, cs.x, sn.x), rope_hi(o.y, qreg.y, cs.y, sn.y), rope_hi(o.z, qreg.z, cs.z, sn.z), rope_hi(o.w, qreg.w, cs.w, sn.w));
    }
  };
  const bool writer = ROPE && head % (H / KV) == 0; // one query head per KV head stores the new k and v
  bool q_stored = false;
  __nv_bfloat16 *kb = k_cache + ((int64_t)b * KV + kvh) * max_seq * ATT_HD, *vb = v_cache + ((int64_t)b * KV + kvh) * max_seq * ATT_HD;
  float m = -INFINITY, l = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int base = c0 + warp * 32; base < c1; base += ATT_WARPS * 32) {
    const int p = base + lane;
    const int cnt = min(32, c1 - base);
    float s = -INFINITY;
    // Everything the run needs from memory is requested at once, so that the run costs one trip to memory and not
    // several in a row: the 32 k rows (8 KB, contiguous in the cache) with coalesced 16-byte loads, and this lane's
    // four dimensions of the 32 v rows (coalesced 256-byte rows).
    uint4 kv[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const int idx = i * 32 + lane, row = idx >> 4, ch = idx & 15;
      kv[i] = make_uint4(0, 0, 0, 0);
      if (row < cnt && base + row != fresh) kv[i] = *reinterpret_cast<const uint4 *>(kb + (int64_t)(base + row) * ATT_HD + ch * 8);
    }
    uint2 vr[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
      vr[j] = make_uint2(0, 0);
      if (j < cnt && base + j != fresh) vr[j] = *reinterpret_cast<const uint2 *>(vb + (int64_t)(base + j) * ATT_HD + lane * 4);
    }
    if (!waited) { // ROPE form: from here on qkv is read
      pdl_wait();
      waited = true;
    }
    if (ROPE && !q_stored) load_rotate_q();
    if (ROPE && fresh >= base && fresh < base + cnt) { // the new row: rotated k and plain v from qkv, rounded to the cache's bf16
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const int idx = i * 32 + lane, row = idx >> 4, ch = idx & 15;
        if (base + row == fresh) { // elements 8 ch .. 8 ch + 7 of the row
          const float *ksrc = q + ((int64_t)b * (H + 2 * KV) + H + kvh) * ATT_HD;
          const int d0 = (ch & 7) * 8;
          float x1[8], x2[8], c[8], sn8[8];
          load8(ksrc + d0, x1);
          load8(ksrc + d0 + ATT_HD / 2, x2);
          load8(cos_t + (int64_t)last * (ATT_HD / 2) + d0, c);
          load8(sin_t + (int64_t)last * (ATT_HD / 2) + d0, sn8);
          __nv_bfloat162 r[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const float a = ch < 8 ? rope_lo(x1[2 * e], x2[2 * e], c[2 * e], sn8[2 * e]) : rope_hi(x1[2 * e], x2[2 * e], c[2 * e], sn8[2 * e]);
            const float bb = ch < 8 ? rope_lo(x1[2 * e + 1], x2[2 * e + 1], c[2 * e + 1], sn8[2 * e + 1]) : rope_hi(x1[2 * e + 1], x2[2 * e + 1], c[2 * e + 1], sn8[2 * e + 1]);
            r[e] = __halves2bfloat162(__float2bfloat16_rn(a), __float2bfloat16_rn(bb));
          }
          kv[i] = *reinterpret_cast<const uint4 *>(r);
          if (writer) *reinterpret_cast<uint4 *>(kb + (int64_t)fresh * ATT_HD + ch * 8) = kv[i];
        }
      }
      const float4 vv = *reinterpret_cast<const float4 *>(q + ((int64_t)b * (H + 2 * KV) + H + KV + kvh) * ATT_HD + lane * 4);
      __nv_bfloat162 r2[2] = {__halves2bfloat162(__float2bfloat16_rn(vv.x), __float2bfloat16_rn(vv.y)), __halves2bfloat162(__float2bfloat16_rn(vv.z), __float2bfloat16_rn(vv.w))};
      const uint2 vnew = *reinterpret_cast<const uint2 *>(r2);
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (base + j == fresh) vr[j] = vnew;
      if (writer) *reinterpret_cast<uint2 *>(vb + (int64_t)fresh * ATT_HD + lane * 4) = vnew;
    }
    // the k rows are turned through shared memory, so that each lane can then read ITS row: a lane reading its own
    // row straight from global memory makes every load instruction touch 32 different lines
    __syncwarp();
    if (!q_stored) {
      *reinterpret_cast<float4 *>(&s_q[warp][lane * 4]) = make_float4(qreg.x * scale, qreg.y * scale, qreg.z * scale, qreg.w * scale);
      q_stored = true;
    }
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const int idx = i * 32 + lane, row = idx >> 4, ch = idx & 15;
      *reinterpret_cast<uint4 *>(&s_k[warp][row][ch * 8]) = kv[i];
    }
    __syncwarp();
    if (p < c1) {
      float d = 0.f;
#pragma unroll
      for (int c = 0; c < 16; c++) {
        const uint4 kr = *reinterpret_cast<const uint4 *>(&s_k[warp][lane][c * 8]);
        const float4 qa = *reinterpret_cast<const float4 *>(&s_q[warp][c * 8]), qb = *reinterpret_cast<const float4 *>(&s_q[warp][c * 8 + 4]);
        const float2 k0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&kr.x)), k1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&kr.y));
        const float2 k2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&kr.z)), k3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&kr.w));
        d += qa.x * k0.x + qa.y * k0.y + qa.z * k1.x + qa.w * k1.y + qb.x * k2.x + qb.y * k2.y + qb.z * k3.x + qb.w * k3.y;
      }
      s = d;
    }
    const float mn = fmaxf(m, warp_max(s));
    const float pw = s == -INFINITY ? 0.f : __expf(s - mn), corr = m == -INFINITY ? 0.f : __expf(m - mn);
    l = l * corr + warp_sum(pw);
    acc = make_float4(acc.x * corr, acc.y * corr, acc.z * corr, acc.w * corr);
#pragma unroll
    for (int j = 0; j < 32; j++) { // rows past the end have weight 0 and zero values
      const float w = __shfl_sync(0xffffffffu, pw, j);
      const float2 v01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&vr[j].x)), v23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&vr[j].y));
      acc.x += w * v01.x, acc.y += w * v01.y, acc.z += w * v23.x, acc.w += w * v23.y;
    }
    m = mn;
  }
  if (!waited) pdl_wait(); // warps without a run of their own: the grid must not complete before its predecessor
  if (lane == 0) s_m[warp] = m, s_l[warp] = l;
  *reinterpret_cast<float4 *>(&s_acc[warp][lane * 4]) = acc;
  __syncthreads();
  float *group = part + ((int64_t)b * H + head) * ATT_GROUP;
  float *rec = group + 4 + split * ATT_REC;
  if (warp == 0) { // merge the CTA's warps; lane owns dims 4*lane..
    float gm = s_m[0], gl = s_l[0];
    float4 ga = *reinterpret_cast<const float4 *>(&s_acc[0][lane * 4]);
#pragma unroll
    for (int w = 1; w < ATT_WARPS; w++) online_merge(gm, gl, ga, s_m[w], s_l[w], *reinterpret_cast<const float4 *>(&s_acc[w][lane * 4]));
    if (nsplit == 1) {
      *reinterpret_cast<float4 *>(out + ((int64_t)b * H + head) * ATT_HD + lane * 4) = make_float4(ga.x / gl, ga.y / gl, ga.z / gl, ga.w / gl);
      return;
    }
    if (lane == 0) rec[0] = gm, rec[1] = gl;
    rec[2 + lane * 4 + 0] = ga.x, rec[2 + lane * 4 + 1] = ga.y, rec[2 + lane * 4 + 2] = ga.z, rec[2 + lane * 4 + 3] = ga.w;
    __threadfence();
    __syncwarp();
    if (lane == 0) s_last = atomicInc(reinterpret_cast<unsigned int *>(group), nsplit - 1) == (unsigned)(nsplit - 1);
    __syncwarp();
    if (!s_last) return;
    __threadfence();
    const float *r0 = group + 4;
    gm = -INFINITY, gl = 0.f, ga = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sidx = 0; sidx < nsplit; sidx++) {
      const volatile float *r = r0 + sidx * ATT_REC;
      online_merge(gm, gl, ga, r[0], r[1], make_float4(r[2 + lane * 4], r[3 + lane * 4], r[4 + lane * 4], r[5 + lane * 4]));
    }
    *reinterpret_cast<float4 *>(out + ((int64_t)b * H + head) * ATT_HD + lane * 4) = make_float4(ga.x / gl, ga.y / gl, ga.z / gl, ga.w / gl);
  }
}

} // namespace
} // namespace xnq

using namespace xnq;

extern "C" {

static int check_image(const char *who, const void *image, int act_dtype, int64_t k) {
  if (!image) return XNQ_OK;
  if (act_dtype != XNQ_Q8_0 && act_dtype != XNQ_Q8K && act_dtype != XNQ_ACT_OPERAND)
    return fail(XNQ_ERR_DTYPE, "%s: %d is not an activation block format (Q8_0=8, Q8K=15) nor XNQ_ACT_OPERAND", who, act_dtype);
  const int blk = act_dtype == XNQ_Q8_0 ? QK : QK_K;
  if (k % blk) return fail(XNQ_ERR_SHAPE, "%s: row length %lld is not a multiple of the %d-value block", who, (long long)k, blk);
  if (reinterpret_cast<uintptr_t>(image) & 255) return fail(XNQ_ERR_ALIGN, "%s: the activation image must be 256-byte aligned", who);
  return XNQ_OK;
}

int xnq_add_rmsnorm(float *x, const float *delta, int delta_parts, const float *weight, float eps, float *out, void *act_image, int act_dtype, int64_t rows,
                    int64_t d, void *stream) {
  clear_error();
  if (!x || !weight || (!out && !act_image)) return fail(XNQ_ERR_NULL, "add_rmsnorm: NULL argument");
  if (rows < 0 || d <= 0 || d % 8 || (delta && delta_parts < 1))
    return fail(XNQ_ERR_SHAPE, "add_rmsnorm: rows = %lld, d = %lld (a multiple of 8), delta_parts = %d", (long long)rows, (long long)d, delta_parts);
  if (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) return fail(XNQ_ERR_ALIGN, "add_rmsnorm: pointers must be 16-byte aligned");
  int rc = check_image("add_rmsnorm", act_image, act_dtype, d);
  if (rc != XNQ_OK) return rc;
  if (rows == 0) return XNQ_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)rows), block(256);
  if (!act_image) XNQ_CUDA(launch_pdl(add_rmsnorm_kernel<0>, grid, block, 0, s, x, delta, delta_parts, weight, eps, out, nullptr, rows, (int)d));
  else if (act_dtype == XNQ_ACT_OPERAND) {
    if (rows > IMMA_MAX_M) return fail(XNQ_ERR_SIZE, "add_rmsnorm: an operand image holds at most %lld rows", (long long)IMMA_MAX_M);
    XNQ_CUDA(launch_pdl(add_rmsnorm_kernel<ACT_OPERAND>, grid, block, 0, s, x, delta, delta_parts, weight, eps, out, act_image, rows, (int)d));
  } else if (act_dtype == XNQ_Q8_0) XNQ_CUDA(launch_pdl(add_rmsnorm_kernel<XNQ_Q8_0>, grid, block, 0, s, x, delta, delta_parts, weight, eps, out, act_image, rows, (int)d));
  else XNQ_CUDA(launch_pdl(add_rmsnorm_kernel<XNQ_Q8K>, grid, block, 0, s, x, delta, delta_parts, weight, eps, out, act_image, rows, (int)d));
  count_launch();
  return XNQ_OK;
}

int xnq_swiglu(const float *gate_up, float *out, void *act_image, int act_dtype, int64_t rows, int64_t f, void *stream) {
  clear_error();
  if (!gate_up || (!out && !act_image)) return fail(XNQ_ERR_NULL, "swiglu: NULL argument");
  if (rows < 0 || f <= 0 || f % 8) return fail(XNQ_ERR_SHAPE, "swiglu: rows = %lld, f = %lld (f must be a multiple of 8)", (long long)rows, (long long)f);
  if (act_image && f % 256) return fail(XNQ_ERR_SHAPE, "swiglu: f = %lld must be a multiple of 256 when an activation image is written", (long long)f);
  if (((uintptr_t)gate_up | (uintptr_t)out) & 15) return fail(XNQ_ERR_ALIGN, "swiglu: pointers must be 16-byte aligned");
  int rc = check_image("swiglu", act_image, act_dtype, f);
  if (rc != XNQ_OK) return rc;
  if (rows == 0) return XNQ_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((rows * f / 8 + 255) / 256);
  if (!act_image) XNQ_CUDA(launch_pdl(swiglu_kernel<0>, dim3(grid), dim3(256), 0, s, gate_up, out, nullptr, rows, (int)f));
  else if (act_dtype == XNQ_ACT_OPERAND) {
    if (rows > IMMA_MAX_M) return fail(XNQ_ERR_SIZE, "swiglu: an operand image holds at most %lld rows", (long long)IMMA_MAX_M);
    XNQ_CUDA(launch_pdl(swiglu_kernel<ACT_OPERAND>, dim3(grid), dim3(256), 0, s, gate_up, out, act_image, rows, (int)f));
  } else if (act_dtype == XNQ_Q8_0) XNQ_CUDA(launch_pdl(swiglu_kernel<XNQ_Q8_0>, dim3(grid), dim3(256), 0, s, gate_up, out, act_image, rows, (int)f));
  else XNQ_CUDA(launch_pdl(swiglu_kernel<XNQ_Q8K>, dim3(grid), dim3(256), 0, s, gate_up, out, act_image, rows, (int)f));
  count_launch();
  return XNQ_OK;
}

int xnq_rope_kv_store(const float *qkv, const float *cos_table, const float *sin_table, const long long *pos_dev, float *q_out, void *k_cache,
                      void *v_cache, int64_t batch, int heads, int kv_heads, int head_dim, int64_t max_seq, void *stream) {
  clear_error();
  if (!qkv || !cos_table || !sin_table || !pos_dev || !q_out || !k_cache || !v_cache) return fail(XNQ_ERR_NULL, "rope_kv_store: NULL argument");
  if (batch < 0 || heads < 1 || kv_heads < 1 || head_dim < 2 || head_dim % 2 || head_dim > 2048 || max_seq < 1)
    return fail(XNQ_ERR_SHAPE, "rope_kv_store: batch %lld heads %d kv_heads %d head_dim %d max_seq %lld", (long long)batch, heads, kv_heads, head_dim, (long long)max_seq);
  if (batch == 0) return XNQ_OK;
  XNQ_CUDA(launch_pdl(rope_store_kernel, dim3(heads + 2 * kv_heads, (unsigned)batch), dim3(head_dim / 2), 0, static_cast<cudaStream_t>(stream), qkv, cos_table,
                      sin_table, pos_dev, q_out, static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache), heads, kv_heads, head_dim, (int)max_seq));
  count_launch();
  return XNQ_OK;
}

int xnq_embed_rows(const void *table_bf16, const long long *tokens, float *x, int64_t rows, int64_t d, int64_t vocab, void *stream) {
  clear_error();
  if (!table_bf16 || !tokens || !x) return fail(XNQ_ERR_NULL, "embed_rows: NULL argument");
  if (rows < 0 || d <= 0 || d % 8 || vocab < 1) return fail(XNQ_ERR_SHAPE, "embed_rows: rows = %lld, d = %lld (a multiple of 8), vocab = %lld", (long long)rows, (long long)d, (long long)vocab);
  if (((uintptr_t)table_bf16 | (uintptr_t)x) & 15) return fail(XNQ_ERR_ALIGN, "embed_rows: pointers must be 16-byte aligned");
  if (rows == 0) return XNQ_OK;
  embed_rows_kernel<<<dim3((unsigned)rows), dim3(256), 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16 *>(table_bf16), tokens, x, (int)d, (long long)vocab);
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int xnq_argmax_advance(const float *logits, int64_t rows, int64_t n, long long *tokens, long long *pos, void *stream) {
  clear_error();
  if (!logits || !tokens) return fail(XNQ_ERR_NULL, "argmax_advance: NULL argument");
  if (rows < 0 || n < 1) return fail(XNQ_ERR_SHAPE, "argmax_advance: rows = %lld, n = %lld", (long long)rows, (long long)n);
  if (rows == 0) return XNQ_OK;
  XNQ_CUDA(launch_pdl(argmax_advance_kernel, dim3((unsigned)rows), dim3(256), 0, static_cast<cudaStream_t>(stream), logits, (long long)n, tokens, pos));
  count_launch();
  return XNQ_OK;
}

size_t xnq_attn_decode_workspace_bytes(int64_t batch, int heads) {
  if (batch <= 0 || heads <= 0) return 0;
  return (size_t)batch * heads * ATT_GROUP * sizeof(float);
}

int xnq_attn_decode(const float *q, const void *k_cache, const void *v_cache, const long long *pos_dev, float *out, int64_t batch, int heads,
                    int kv_heads, int head_dim, int64_t max_seq, void *workspace, size_t ws_bytes, void *stream) {
  clear_error();
  if (!q || !k_cache || !v_cache || !pos_dev || !out) return fail(XNQ_ERR_NULL, "attn_decode: NULL argument");
  if (head_dim != ATT_HD) return fail(XNQ_ERR_UNSUPPORTED, "attn_decode: head_dim %d (this kernel is written for %d)", head_dim, ATT_HD);
  if (batch < 0 || heads < 1 || kv_heads < 1 || heads % kv_heads || max_seq < 1)
    return fail(XNQ_ERR_SHAPE, "attn_decode: batch %lld heads %d kv_heads %d max_seq %lld", (long long)batch, heads, kv_heads, (long long)max_seq);
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out | (uintptr_t)workspace) & 15) return fail(XNQ_ERR_ALIGN, "attn_decode: pointers must be 16-byte aligned");
  if (batch == 0) return XNQ_OK;
  const size_t need = xnq_attn_decode_workspace_bytes(batch, heads);
  if (!workspace || ws_bytes < need) return fail(XNQ_ERR_SIZE, "attn_decode: workspace has %zu bytes, needs %zu (zero it once after allocating)", ws_bytes, need);
  int splits = (int)(296 / (batch * heads));
  splits = splits < 1 ? 1 : (splits > ATT_MAX_SPLITS ? ATT_MAX_SPLITS : splits);
  float *part = static_cast<float *>(workspace);
  XNQ_CUDA(launch_pdl(attn_decode_kernel<false>, dim3(heads, (unsigned)batch, splits), dim3(ATT_WARPS * 32), 0, static_cast<cudaStream_t>(stream), q,
                      static_cast<__nv_bfloat16 *>(const_cast<void *>(k_cache)), static_cast<__nv_bfloat16 *>(const_cast<void *>(v_cache)), pos_dev, out, part, heads,
                      kv_heads, (int)max_seq, 1.0f / sqrtf((float)head_dim), static_cast<const float *>(nullptr), static_cast<const float *>(nullptr)));
  count_launch();
  return XNQ_OK;
}

int xnq_rope_attn_decode(const float *qkv, const float *cos_table, const float *sin_table, const long long *pos_dev, void *k_cache, void *v_cache, float *out,
                         int64_t batch, int heads, int kv_heads, int head_dim, int64_t max_seq, void *workspace, size_t ws_bytes, void *stream) {
  clear_error();
  if (!qkv || !cos_table || !sin_table || !pos_dev || !k_cache || !v_cache || !out) return fail(XNQ_ERR_NULL, "rope_attn_decode: NULL argument");
  if (head_dim != ATT_HD) return fail(XNQ_ERR_UNSUPPORTED, "rope_attn_decode: head_dim %d (this kernel is written for %d)", head_dim, ATT_HD);
  if (batch < 0 || heads < 1 || kv_heads < 1 || heads % kv_heads || max_seq < 1)
    return fail(XNQ_ERR_SHAPE, "rope_attn_decode: batch %lld heads %d kv_heads %d max_seq %lld", (long long)batch, heads, kv_heads, (long long)max_seq);
  if (((uintptr_t)qkv | (uintptr_t)cos_table | (uintptr_t)sin_table | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out | (uintptr_t)workspace) & 15)
    return fail(XNQ_ERR_ALIGN, "rope_attn_decode: pointers must be 16-byte aligned");
  if (batch == 0) return XNQ_OK;
  const size_t need = xnq_attn_decode_workspace_bytes(batch, heads);
  if (!workspace || ws_bytes < need) return fail(XNQ_ERR_SIZE, "rope_attn_decode: workspace has %zu bytes, needs %zu (zero it once after allocating)", ws_bytes, need);
  int splits = (int)(296 / (batch * heads));
  splits = splits < 1 ? 1 : (splits > ATT_MAX_SPLITS ? ATT_MAX_SPLITS : splits);
  XNQ_CUDA(launch_pdl(attn_decode_kernel<true>, dim3(heads, (unsigned)batch, splits), dim3(ATT_WARPS * 32), 0, static_cast<cudaStream_t>(stream), qkv,
                      static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache), pos_dev, out, static_cast<float *>(workspace), heads, kv_heads,
                      (int)max_seq, 1.0f / sqrtf((float)head_dim), cos_table, sin_table));
  count_launch();
  return XNQ_OK;
}

} // extern "C"

namespace xnq {
int decoder_status(unsigned int *bits) {
  XNQ_CUDA(cudaMemcpyFromSymbol(bits, g_decoder_status, sizeof(*bits)));
  return XNQ_OK;
}
int decoder_ops_init() {
  unsigned int zero = 0;
  XNQ_CUDA(cudaMemcpyToSymbol(g_decoder_status, &zero, sizeof(zero)));
  return XNQ_OK;
}
} // namespace xnq
