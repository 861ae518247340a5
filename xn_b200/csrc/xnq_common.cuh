// Shared declarations of the xnq library: device weight handle, activation workspace views,
// error plumbing, launch entry points of each translation unit. sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/xnq.h"

namespace xnq {

constexpr int QK = 32;    // elements per Q4_0 / Q8_0 block (k_quants.rs:14-19)
constexpr int QK_K = 256; // elements per K-quant super-block (k_quants.rs:11)

// ------------------------------------------------------------------------------------------------
// error plumbing: thread-local message + status code
// ------------------------------------------------------------------------------------------------
int fail(int code, const char *fmt, ...);
void clear_error();
#define XNQ_CUDA(expr)                                                                              \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess)                                                                         \
      return ::xnq::fail(XNQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));            \
  } while (0)

inline int type_size(int dt) {
  switch (dt) {
    case XNQ_F32: return 4;
    case XNQ_F16: return 2;
    case XNQ_BF16: return 2;
    case XNQ_Q4_0: return 18;
    case XNQ_Q4_1: return 20;
    case XNQ_Q5_0: return 22;
    case XNQ_Q5_1: return 24;
    case XNQ_Q8_0: return 34;
    case XNQ_Q8_1: return 36;
    case XNQ_Q2K: return 84;
    case XNQ_Q3K: return 110;
    case XNQ_Q4K: return 144;
    case XNQ_Q5K: return 176;
    case XNQ_Q6K: return 210;
    case XNQ_Q8K: return 292;
  }
  return -1;
}
inline int block_size(int dt) {
  switch (dt) {
    case XNQ_F32:
    case XNQ_F16:
    case XNQ_BF16: return 1;
    case XNQ_Q4_0:
    case XNQ_Q4_1:
    case XNQ_Q5_0:
    case XNQ_Q5_1:
    case XNQ_Q8_0:
    case XNQ_Q8_1: return QK;
    case XNQ_Q2K:
    case XNQ_Q3K:
    case XNQ_Q4K:
    case XNQ_Q5K:
    case XNQ_Q6K:
    case XNQ_Q8K: return QK_K;
  }
  return -1;
}
// the four formats with their own device layouts and fast kernels, and the six held as canonical blocks (xnq_generic.cu)
inline bool is_fast_dtype(int dt) { return dt == XNQ_Q4_0 || dt == XNQ_Q8_0 || dt == XNQ_Q4K || dt == XNQ_Q6K; }
bool is_generic_dtype(int dt);
inline bool is_weight_dtype(int dt) { return is_fast_dtype(dt) || is_generic_dtype(dt); }
inline bool is_float_dtype(int dt) { return dt == XNQ_F32 || dt == XNQ_F16 || dt == XNQ_BF16; }
// GgmlType::VecDotType (k_quants.rs:210,310,405,511,615,883,1046,1321,1510,1727)
inline int act_dtype_for(int wdt) {
  switch (wdt) {
    case XNQ_Q4_0:
    case XNQ_Q5_0:
    case XNQ_Q8_0: return XNQ_Q8_0;
    case XNQ_Q4_1:
    case XNQ_Q5_1: return XNQ_Q8_1;
    default: return XNQ_Q8K;
  }
}

// ------------------------------------------------------------------------------------------------
// Device layout of a weight (or N-shard): what the kernels read.
//
//  Q4_0 : qs  [n][k/32][16]  nibble bytes exactly as in the GGUF block (16-byte chunks now aligned)
//         d   [n][dstride]   f16 block scales
//  Q8_0 : qs  [n][k]         int8 codes
//         d   [n][dstride]   f16 block scales
//  Q4_K : qs  = the 144-byte super-blocks in GGUF order (144 = 9 x 16 B: already aligned); only the
//               12 scale bytes are re-packed into four 24-bit per-group fields (xnq_unpack.cuh)
//  Q6_K : qs  [n][k/256][128] ql bytes,  qh [n][k/256][64],  sc [n][k/256][16] int8,
//         d   [n][dstride]   f16 super-block scales
// dstride (elements) is the scale count per row rounded up to 8, so every row of d starts 16-byte
// aligned. Total bytes equal the GGUF bytes (plus that padding).
// ------------------------------------------------------------------------------------------------
struct WeightView {
  int dtype;
  int64_t n; // rows held
  int64_t k;
  int64_t dstride;
  const uint8_t *qs;
  const uint8_t *qh;
  const int8_t *sc;
  const __half *d;
};

// Planar device layout of quantized activations (the matmul scratch):
//  q     [m][k]        int8 codes
//  d     [m][k/blk]    f32 block scale (Q8_0: the f16-rounded scale widened, so dots use exactly
//                      the value the reference reads back from the block; Q8_K: the f32 scale)
//  bsum  [m][k/16]     int16 sums of 16 codes (BlockQ8K::bsums; for Q8_0 blocks the same sums, used
//                      to fold Q4_0's -8 offset)
struct ActView {
  int act_dtype; // XNQ_Q8_0 or XNQ_Q8K
  int64_t m, k;
  int8_t *q;
  float *d;
  int16_t *bsum;
};

// Destination of an N-sharded matmul whose output slices are gathered on every rank by peer stores.
// dst[r] is rank r's gathered-output buffer for this call (dst[rank] is local, the others are peer
// mappings of the same allocation on the other GPUs); this rank writes columns [col0, col0 + n) of
// every row into all of them. flag[r] is the address, inside rank r's mapping, of the word that
// carries THIS rank's epoch (flag[rank] is the local word); ctl is local: {epochs sent, unused, CTAs done, late-peer bits}.
constexpr int XNQ_MAX_RANKS = 8;
struct GatherArgs {
  void *dst[XNQ_MAX_RANKS];
  unsigned int *flag[XNQ_MAX_RANKS];
  unsigned int *ctl;
  int world, rank;
  int cta_fence_gpu; // 1: CTAs order their stores before the arrival count with a gpu-scope fence; the last CTA's system-scope release carries them on
  int defer_wait;    // 1: the kernel publishes its epoch and retires; the peers' columns are awaited later (xnq_comm_wait)
  int64_t col0, ld; // first column this rank produces; row stride of the gathered buffer (elements)
};

#ifdef __CUDACC__
constexpr unsigned long long GATHER_WAIT_LIMIT_NS = 4000000000ull; // a peer that has not published within 4 s is reported, not awaited

// Called by one whole warp of each CTA after a CTA-wide barrier that follows the CTA's stores into the
// gathered buffers. The last CTA of the launch advances this rank's epoch, stores it with release
// semantics at system scope into every peer's epoch row, and then waits until every peer's epoch in
// the local row has reached the same count: when the launch retires, the gathered buffer of this
// rank is complete. The wait is bounded; a late peer sets its bit in ctl[3] and the kernel returns.
// Ordering: the CTA's stores precede its barrier; the calling thread then fences at gpu scope and counts
// its arrival (a release pattern the last CTA's atomic + system-scope fence acquires), and the last
// CTA's release store at system scope carries every CTA's stores with it (causality order is
// cumulative across scopes). A system-scope fence in every CTA is not needed and costs about 3 us per
// launch; the "gather_cta_fence" option (0) brings it back for comparison.
__device__ __forceinline__ void gather_await_peer(const GatherArgs &g, unsigned int epoch, int lane);
__device__ __forceinline__ void gather_publish_and_wait(const GatherArgs &g) {
  // called by the 32 lanes of ONE warp of each CTA, after the CTA-wide barrier that follows its stores
  const int lane = threadIdx.x & 31;
  unsigned int last = 0, epoch = 0;
  if (lane == 0) {
    if (g.cta_fence_gpu) __threadfence();
    else __threadfence_system();
    if (atomicAdd(g.ctl + 2, 1u) == gridDim.x - 1) {
      g.ctl[2] = 0;
      epoch = g.ctl[0] + 1;
      g.ctl[0] = epoch;
      last = g.ctl[3] ? 2u : 1u; // 2: a peer was already late once, later launches publish but do not wait again
      __threadfence_system();
    }
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return;
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  // lane p talks to rank p: all peers are told, and all peers are awaited, at the same time
  const bool peer = lane < g.world && lane != g.rank;
  if (peer) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(g.flag[lane]), "r"(epoch) : "memory");
  if (last == 2u || !peer || g.defer_wait) return;
  gather_await_peer(g, epoch, lane);
}
// lane p (a peer's rank) waits, bounded, until that peer's epoch word in the local row has reached `epoch`
__device__ __forceinline__ void gather_await_peer(const GatherArgs &g, unsigned int epoch, int lane) {
  const unsigned int *mine = g.flag[g.rank] - g.rank + lane; // this peer's word in the local epoch row
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - epoch) >= 0) break;
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    if (t - t0 > GATHER_WAIT_LIMIT_NS) {
      atomicOr(g.ctl + 3, 1u << lane);
      break;
    }
  }
}
#endif

size_t act_workspace_bytes(int64_t m, int64_t k, int act_dtype);
ActView act_view(void *workspace, int64_t m, int64_t k, int act_dtype);

} // namespace xnq

struct xnq_weight {
  int device;
  int64_t n_total, row0;
  xnq::WeightView v;
  void *base;    // single device allocation behind v
  size_t bytes;  // its size
  float wscale;  // power of two that brings the largest |weight| into (2^9, 2^10] for the fp16 prefill path
  // host-call staging (xnq_linear_forward_host)
  void *stage_dev;
  size_t stage_dev_bytes;
  void *stage_host;
  size_t stage_host_bytes;
};

namespace xnq {

// launch accounting + per-kernel event timing (xnq_api.cu)
void count_launch(int n = 1);

// ---- programmatic dependent launch ---------------------------------------------------------------------------
// Every kernel of the decode step is launched with programmatic stream serialization: it lets its successor in the
// stream start (pdl_launch_dependents, first thing) while it is still running, and itself touches nothing an earlier
// kernel may still write or read before pdl_wait() returns (the earlier grids have completed and their writes are
// visible). What a kernel does before pdl_wait() is limited to set-up and to reading immutable data (weights), so
// results are exactly those of plain stream order; what is gained is the launch latency of every kernel and, for the
// weight-streaming kernels, the start of their stream. Every CTA executes pdl_wait() before it exits, so a grid never
// completes before its predecessors.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&...args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
void profile_mark(cudaStream_t s, bool start);

// xnq_layout.cu
int launch_relayout(const WeightView &dst, const uint8_t *canonical_dev, cudaStream_t s);   // GGUF -> device layout
int launch_to_canonical(const WeightView &src, uint8_t *canonical_dev, cudaStream_t s);     // device layout -> GGUF
int launch_dequantize(const WeightView &w, int out_dtype, void *dst, cudaStream_t s);
// formats held as canonical blocks (xnq_generic.cu)
int generic_init(int device);
int launch_generic_dequantize(const WeightView &w, int out_dtype, void *dst, cudaStream_t s);
int launch_quantize_q8_1(const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx, void *dst, cudaStream_t s);
size_t generic_workspace_bytes(const WeightView &w, int64_t m);
int launch_generic_matmul(const WeightView &w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy, void *workspace,
                          cudaStream_t s);
int layout_init(int device);

// xnq_quantize_act.cu
int launch_quantize_act_blocks(int act_dtype, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx,
                               void *dst_blocks, cudaStream_t s);
int launch_quantize_act_planar(const ActView &a, const void *x, int x_dtype, int64_t ldx, cudaStream_t s);
int quantize_init(int device);

// xnq_quantize_weight.cu: dense f32 [n, k] on the device -> canonical GGUF blocks on the device
int launch_quantize_weight(int dtype, const float *x, int64_t n, int64_t k, void *blocks, cudaStream_t s);

// xnq_matvec.cu  (m <= 16)
constexpr int MATVEC_MAX_M = 16;
int launch_matvec(const WeightView &w, const ActView &a, void *y, int y_dtype, int64_t ldy, cudaStream_t s);
int matvec_init(int device);
// activation rows one matvec launch can stage in shared memory for this k (0: k is too large)
int64_t matvec_rows_per_pass(int wdtype, int64_t k);

// xnq_matvec_mma.cu  (5 <= m <= 16, Q4_K: integer tensor-core MMAs)
int64_t matvec_mma_rows_per_pass(const WeightView &w, int y_dtype); // 0: not served
int launch_matvec_mma(const WeightView &w, const ActView &a, void *y, int y_dtype, int64_t ldy, cudaStream_t s);
bool matvec_mma_accumulates_in_y(const WeightView &w, int64_t m); // k split between CTAs that add into y atomically
int matvec_mma_init(int device);
// rows per launch of the small-batch path that xnq_matmul_t takes for this weight, and which kernel that is
int64_t small_batch_pass(const xnq_weight *w, int64_t m, int y_dtype, bool *use_mma);

// xnq_matvec_ring.cu  (m == 1: persistent bulk-copy ring kernel; quantizes x in its prologue when k <= 4096)
bool matvec_tma_supported(const WeightView &w, int64_t m);
bool matvec_tma_wants_image(const WeightView &w); // k above 4096: the activations must come as an activation image
void matvec_hint_next(const xnq_weight *w);        // the weight the calling thread's stream multiplies next (one-shot)
// g != nullptr: results go to column col0 + row of every rank's gathered buffer (y is ignored)
// Residual add + RMSNorm applied by the one-row matvec in its prologue (x_in null: none). Every CTA forms the row
// x_in + sum of the `parts` summands, normalises it and quantizes it for itself; CTA 0 also writes the new residual to
// x_out, which must not be x_in (other CTAs may still be reading x_in).
struct NormArgs {
  const float *x_in = nullptr;
  const float *delta = nullptr; // [parts][k] summands, or null
  int parts = 0;
  const float *weight = nullptr;
  float eps = 0.f;
  float *x_out = nullptr;
  // When the summands are the output of a gather that was left un-awaited (xnq_comm_set_deferred): the kernel first awaits,
  // bounded, that every peer has published as many gathers as this rank (wait_ctl[0]); wait_row is this rank's epoch row.
  unsigned int *wait_ctl = nullptr;
  const unsigned int *wait_row = nullptr;
  int wait_world = 0, wait_rank = 0;
};
int comm_fill_wait(const xnq_comm *c, NormArgs *na); // xnq_comm.cu
int launch_matvec_tma(const WeightView &w, const void *x, int x_dtype, void *y, int y_dtype, cudaStream_t s, const GatherArgs *g = nullptr,
                      const NormArgs *norm = nullptr);
bool matvec_tma_enabled(); // the "matvec_tma" library option
int gather_cta_fence_scope(); // the "gather_cta_fence" library option
// shared argument checks of the matmul entries (dtype, leading dimension, 16-byte row alignment)
int check_activations(const char *who, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx);
int matvec_tma_init(int device);
int matvec_status(unsigned int *bits);
int matvec_check_record(unsigned long long out[8]);

// xnq_imma.cu  (2 <= m: tcgen05 kind::i8, exact integer block sums; Q4_0 / Q8_0 / Q4_K)
bool imma_supported(const WeightView &w, int64_t m);
size_t imma_workspace_bytes(int64_t m, int64_t k, int64_t n);
int launch_imma(const WeightView &w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy, void *workspace,
                cudaStream_t s);
int imma_init(int device);
void imma_set_fold(int mode); // Q4_K kernel with the sub-block scales folded into the weight operand: 0 never, 1 where it is faster (17..32 rows), 2 always
int imma_status(unsigned int *bits);
int decoder_ops_init();
int decoder_status(unsigned int *bits); // 1 rope/store, 2 attention: a position outside [0, max_seq)
// Activation OPERAND image (XNQ_ACT_OPERAND): up to 64 rows quantized to Q8_K and laid out as the integer tensor-core kernel reads them,
// so that a producer (add+RMSNorm, SwiGLU) can write them directly and the matmul needs no activation kernel of its own:
//   [4096 bytes]              1024 ticket words of split tiles (zero between matmuls: the kernel puts each word back)
//   [k/256][2][NP x 128]      codes of each 128-k half step, rows 128 bytes apart, 16-byte chunks swizzled with the row (NP = 16 / 32 / 64)
//   [k/256][NP][32]           per step and row: the eight 32-sums as low-7-bit and high bytes (16 bytes), the f32 block scale, 12 bytes of zero
constexpr size_t OPERAND_TICKET_BYTES = 4096;
constexpr int OPERAND_MAX_TILES = 1024;
__host__ __device__ inline int operand_np(int64_t m) { return m <= 16 ? 16 : (m <= 32 ? 32 : 64); }
__host__ __device__ inline size_t operand_bimg_bytes(int np, int64_t k) { return (size_t)(k / 256) * np * 256; }
__host__ __device__ inline size_t operand_image_bytes(int64_t m, int64_t k) { return OPERAND_TICKET_BYTES + (size_t)(k / 256) * operand_np(m) * 288; }
constexpr int64_t IMMA_MAX_M = 64; // batches up to here take the integer tensor-core kernel; larger ones the fp16 one

// xnq_prefill.cu  (m > 64, and Q6_K above 16 rows: tcgen05 / TMEM contraction on fp16 operands)
size_t prefill_workspace_bytes(int64_t m, int64_t k, int64_t n);
int launch_prefill(const WeightView &w, float wscale, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy,
                   void *workspace, cudaStream_t s);
int prefill_init(int device);
int prefill_status(unsigned int *bits);

// largest |dequantized weight| of the tensor, written to *dev_out (a float in device memory)
int launch_max_abs(const WeightView &w, float *dev_out, cudaStream_t s);

// xnq_bias.cu-ish helper in xnq_layout.cu: y[m, n] += bias[n]
int launch_add_bias(float *y, const float *bias, int64_t m, int64_t n, int64_t ldy, cudaStream_t s);

} // namespace xnq
