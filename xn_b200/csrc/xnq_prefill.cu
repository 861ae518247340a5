// Prefill (m > 16): quantized weights x activations as a dense contraction on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in TMEM).
//
//   D[128 weight rows, mt activation rows] += A[128, 64] . B[mt, 64]^T      per k-step of 64
//
//   A  weights of the tile, dequantized by four producer warps (one thread per weight row) from the
//      quantized blocks straight into the 128-byte-swizzled K-major shared-memory image the MMA reads.
//      Every weight is dequantized once per m-tile (mt up to 256 rows).
//   B  activations, prepared once per call by prefill_prepare_acts: quantized to Q8_0 / Q8_K exactly
//      as the reference's quantize_lhs does (k_quants.rs:2015-2026), dequantized, scaled by a power of
//      two per row and stored as fp16 in the same swizzled image, so that one 1-D bulk-async copy
//      (cp.async.bulk, non-multicast) brings a whole stage.
//   D  f32 in tensor memory; four epilogue warps read it back with tcgen05.ld, undo the power-of-two
//      scales and store y.
//
// Operand type. The contraction runs in fp16 (kind::f16 with f16 inputs), not bf16: both have the
// same tensor throughput, and fp16's 11-bit significand keeps the operand rounding 8x smaller: the
// result stays within about 3e-3 of the OUTPUT RMS of the reference's integer-exact CPU result. Under the
// reference's own element-wise metric |g - w| <= tol * max(|w|, 1) that is 1e-2 only while the output rms
// is below about 3; where outputs are larger the integer-exact kernels are the ones that meet it. Range is handled exactly: every activation row and the whole weight tensor are multiplied
// by powers of two that put their maxima near 2^11 / 2^10, and the epilogue divides them out.
//
// k order. A dot product does not care in which order k is visited as long as both operands agree,
// so within a k-step the 64 elements are stored in the order the nibble unpack produces them
// (xnq_prefill.cuh: kperm) and the activation image uses the same order; no shuffles are needed.
//
// Synchronisation. Per stage: a_full (128 producer arrivals), b_full (bulk-copy transaction bytes),
// empty (tcgen05.commit by the MMA thread). Every wait is bounded; on expiry a status bit is set and
// every role falls through to the common exit, where tensor memory is released.
#include <algorithm>
#include <cstring>

#include "xnq_common.cuh"
#include "xnq_quantize_act.cuh"
#include "xnq_prefill_rows.cuh"
#include "xnq_unpack.cuh"

namespace xnq {

__device__ unsigned int g_prefill_status; // sticky: 1 producer wait, 2 loader wait, 4 mma wait, 8 epilogue wait expired

namespace {

constexpr int BK = 64;             // k-step (elements) = one 128-byte swizzle row of fp16
constexpr int TILE_N = 128;        // weight rows per CTA = UMMA M
constexpr int MAX_MT = 256;        // activation rows per CTA = UMMA N
constexpr int GROUP = 256;         // one producer group: two threads per weight row
constexpr int PRODUCERS = 2 * GROUP; // two groups take alternate k-steps, so a warp's per-k-step latency chain is halved
constexpr int LOADER_WARP = PRODUCERS / 32, MMA_WARP = LOADER_WARP + 1;
constexpr int NTHREADS = PRODUCERS + 64; // warps 0-15 producers/epilogue, then the loader warp and the MMA warp
constexpr uint32_t WAIT_LIMIT = 1u << 26; // non-blocking polls (a few ns each): about a second
constexpr int A_STAGE_BYTES = TILE_N * BK * 2; // 16 KB
#ifndef XNQ_PF_NSTAGES
#define XNQ_PF_NSTAGES 4
#endif
#ifndef XNQ_PF_RAW_DEPTH
#define XNQ_PF_RAW_DEPTH 2
#endif
constexpr int NSTAGES = XNQ_PF_NSTAGES; // even: each producer group owns every other A stage
        // A stages (16 KB each)
constexpr int RAW_DEPTH = XNQ_PF_RAW_DEPTH; // own k-steps (every other one) of raw weight bytes a producer thread keeps in flight
constexpr int RAW_SLOT_MAX = 80;   // largest per-thread slot (Q6_K)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int bit) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicOr(&g_prefill_status, bit);
  return false;
}
// for waits that are long by design (a drain warp waiting out a whole main loop): poll at a low rate so the
// poller does not take issue slots from the producer warps of its scheduler
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, unsigned int bit) {
  for (uint32_t i = 0; i < (WAIT_LIMIT >> 4); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(200);
  }
  atomicOr(&g_prefill_status, bit);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}

// ---- tcgen05 wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the mbarrier once every MMA issued so far by this thread has finished reading smem / writing tmem
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
// Fields: start address >> 4 [0,14), leading byte offset >> 4 [16,30) (unused for swizzled K-major),
// stride byte offset >> 4 [32,46), descriptor version 1 [46,48), swizzle mode 2 = 128 B [61,64).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D f32 (bit 4), A/B format (0 = f16) at [7,10) / [10,13), both K-major,
// N >> 3 at [17,23), M >> 4 at [24,29).
__device__ __forceinline__ uint32_t idesc_f16(int umma_n) { return (1u << 4) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24); }

struct PrefillArgs {
  WeightView w;
  const uint8_t *xh;      // activation image: [k-steps][m_pad][64] fp16, swizzled rows, k-step-permuted
  const float *row_unscale; // [m_pad]: 1 / (activation row scale * weight scale)
  void *y;
  int y_dtype;
  int64_t ldy;
  int64_t m, m_pad;
  int ksteps;
  int nstages;            // A (weight) stages
  int b_stages;           // B (activation) stages: deeper, the bulk copy's L2 latency has to be covered
  uint32_t b_stride;      // bytes between B stages (largest mt of the grid x 128, multiple of 1024)
  uint32_t b_off, raw_off; // offsets of the B ring and of the producers' raw rings from the aligned base
  float wscale;           // power of two applied to every dequantized weight
  // persistent kernel: tile t = tile_n * tiles_m + tile_m; work unit u = t * ksteps + kt; CTA c takes units
  // [units * c / G, units * (c + 1) / G), or whole tiles when the output cannot be accumulated atomically
  int tiles_n, tiles_m;
  long long units;
  int whole_tiles;
  unsigned int *tile_cnt; // [tiles] arrival tickets then [tiles] "first partial stored" flags; zeroed by the prepare kernel
};

// Dequantize the 64 weights of k-step `kt` of row `row` and store them as 8 swizzled 16-byte chunks.
// All arithmetic is fp16 on exactly representable integers times an fp16 scale.
using namespace prefill_rows;

__device__ __forceinline__ void zero_half_row(uint32_t dst_row, int hf) { // chunks 4hf..4hf+3, whatever the swizzle
  const int sw = (dst_row >> 7) & 7;
#pragma unroll
  for (int c = 0; c < 4; c++) sts128(dst_row + (((hf * 4 + c) ^ sw) << 4), 0, 0, 0, 0);
}

// Writes one 32-column chunk of an accumulator row block: column j of the chunk is activation row
// m_first + j, this lane's accumulator lane is weight row `row`. MODE: 0 f32 store, 1 f32 atomic add,
// 2 f16 store, 3 bf16 store.
template <int MODE>
__device__ __forceinline__ void drain_chunk(const uint32_t (&v)[32], float ru_lane, void *y, int64_t ldy, int64_t row, int64_t m_first, int64_t m_end,
                                            bool row_ok) {
  // a running pointer and one small count: the few warps that drain have nobody to hide instruction latency
  // behind, so every instruction per column counts
  const int es = MODE <= 1 ? 4 : 2;
  char *yp = static_cast<char *>(y) + (m_first * ldy + row) * es;
  const int64_t step = ldy * es;
  const int nvalid = row_ok ? (int)min((int64_t)32, m_end - m_first) : 0;
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, ru_lane, j);
    if (j < nvalid) {
      if (MODE == 0) *reinterpret_cast<float *>(yp) = val;
      else if (MODE == 1) atomicAdd(reinterpret_cast<float *>(yp), val);
      else if (MODE == 2) *reinterpret_cast<__half *>(yp) = __float2half_rn(val);
      else *reinterpret_cast<__nv_bfloat16 *>(yp) = __float2bfloat16_rn(val);
    }
    yp += step;
  }
}

// ---- the kernel ------------------------------------------------------------------------------------------------
// One CTA per SM walks a contiguous range of the flattened (tile, k-step) space, so all SMs finish
// together whatever the tile count, and a tile whose k-steps are split between CTAs is summed in
// global memory: the first CTA to finish its part stores it and raises the tile's flag, the others add
// theirs atomically after seeing the flag (two to three parts per split tile; f32 output only - other
// output types get whole tiles). The accumulator is double-buffered in tensor memory (2 x 256 columns)
// and drained by four dedicated warps, so the drain of one segment overlaps the MMAs of the next.
// Roles: 16 producer warps in two groups that take alternate k-steps (two threads per weight row, each with a
// private cp.async ring of raw bytes), one activation-loader warp (one bulk copy per stage), one MMA-issuing
// warp, eight drain warps. Stage counters run on across segments.
constexpr int EPI_WARPS = 8; // two per accumulator lane quarter, splitting the columns
constexpr int EPI_WARP0 = MMA_WARP + 1;
constexpr int NTHREADS_SK = NTHREADS + EPI_WARPS * 32;

struct Cursor { // position in the flattened (tile, k-step) space; tile = tile_n * tiles_m + tile_m
  int tile_n, tile_m, kt;
  __device__ __forceinline__ void advance(int steps, int KT, int tiles_m) {
    kt += steps;
    while (kt >= KT) {
      kt -= KT;
      if (++tile_m == tiles_m) {
        tile_m = 0;
        tile_n++;
      }
    }
  }
  __device__ __forceinline__ int tile(int tiles_m) const { return tile_n * tiles_m + tile_m; }
};

template <typename RowT>
__global__ void __launch_bounds__(NTHREADS_SK, 1) prefill_persistent_kernel(PrefillArgs p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ __align__(8) uint64_t bars[4 * 8 + 4]; // a_full, a_empty, b_full, b_empty (8 each), acc_full[2], acc_empty[2]
  __shared__ uint32_t tmem_slot;
  __shared__ unsigned int s_ticket;
  const int S = p.nstages;
  const int SB = p.b_stages;
  const uint32_t a_full = smem_u32(bars), a_empty = a_full + 64, b_full = a_full + 128, b_empty = a_full + 192, acc_full = a_full + 256,
                 acc_empty = a_full + 272;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t a_ring = smem_base, b_ring = smem_base + p.b_off;
  const int KT = p.ksteps;

  // this CTA's range of work units
  long long u0, u1;
  if (p.whole_tiles) {
    const long long T = (long long)p.tiles_n * p.tiles_m;
    u0 = (T * blockIdx.x / gridDim.x) * KT;
    u1 = (T * (blockIdx.x + 1) / gridDim.x) * KT;
  } else {
    u0 = p.units * blockIdx.x / gridDim.x;
    u1 = p.units * (blockIdx.x + 1) / gridDim.x;
  }
  const int nsteps = (int)(u1 - u0);
  const int TM = p.tiles_m;
  const Cursor start{(int)((u0 / KT) / TM), (int)((u0 / KT) % TM), (int)(u0 % KT)};

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mbar_init(a_full + 8 * s, GROUP / 32);
      mbar_init(a_empty + 8 * s, 1);
    }
    for (int s = 0; s < SB; s++) {
      mbar_init(b_full + 8 * s, 1);
      mbar_init(b_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(acc_full + 8 * b, 1);
      mbar_init(acc_empty + 8 * b, EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == LOADER_WARP) {
    tmem_alloc(smem_u32(&tmem_slot), 2 * MAX_MT);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_slot;

  if (warp < PRODUCERS / 32) {
    // ---- producers: group g takes this CTA's steps g, g+2, ... -------------------------------------------
    const int grp = threadIdx.x / GROUP, tg = threadIdx.x % GROUP;
    const int r = tg & (TILE_N - 1), hf = tg >> 7;
    const int sw = r & 7;
    const uint32_t raw_base = smem_base + p.raw_off;
    Cursor cur = start, pre = start;
    cur.advance(grp, KT, TM);
    pre.advance(grp, KT, TM);
#pragma unroll
    for (int j = 0; j < RAW_DEPTH; j++) {
      if (grp + 2 * j < nsteps) {
        const int64_t row = (int64_t)pre.tile_n * TILE_N + r;
        RowT::issue(p.w, row < p.w.n ? row : p.w.n - 1, pre.kt, hf, raw_base + (j * PRODUCERS + threadIdx.x) * RowT::SLOT);
        pre.advance(2, KT, TM);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    int rs = 0;
    bool alive = true;
    for (int i = grp; i < nsteps && alive; i += 2) {
      const int s = i % S;
      const uint32_t round = (uint32_t)(i / S);
      const uint32_t slot = raw_base + (rs * PRODUCERS + threadIdx.x) * RowT::SLOT;
      asm volatile("cp.async.wait_group %0;" ::"n"(RAW_DEPTH - 1) : "memory");
      if (i >= S) {
        int ok = 1;
        if (lane == 0) ok = mbar_wait(a_empty + 8 * s, (round - 1) & 1, 1u) ? 1 : 0;
        __syncwarp();
        alive = __shfl_sync(0xffffffffu, ok, 0) != 0;
      }
      if (!alive) break;
      const int64_t row = (int64_t)cur.tile_n * TILE_N + r;
      const uint32_t dst_row = a_ring + s * A_STAGE_BYTES + r * 128;
      if (row < p.w.n) RowT::store(p.w, slot, cur.kt, hf, p.wscale, dst_row, sw);
      else zero_half_row(dst_row, hf);
      if (i + 2 * RAW_DEPTH < nsteps) {
        const int64_t prow = (int64_t)pre.tile_n * TILE_N + r;
        RowT::issue(p.w, prow < p.w.n ? prow : p.w.n - 1, pre.kt, hf, slot);
        pre.advance(2, KT, TM);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(a_full + 8 * s);
      rs = (rs + 1 == RAW_DEPTH) ? 0 : rs + 1;
      cur.advance(2, KT, TM);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == LOADER_WARP) {
    // ---- activation loader ------------------------------------------------------------------------------
    if (lane == 0) {
      Cursor cur = start;
      int issued = 0;
      for (int i = 0; i < nsteps; i++) {
        const int s = i % SB;
        const uint32_t round = (uint32_t)(i / SB);
        if (round > 0 && !mbar_wait(b_empty + 8 * s, (round - 1) & 1, 2u)) break;
        const int64_t m0 = (int64_t)cur.tile_m * MAX_MT;
        const uint32_t bytes = (uint32_t)min((int64_t)MAX_MT, p.m_pad - m0) * 128;
        mbar_expect_tx(b_full + 8 * s, bytes);
        bulk_g2s(b_ring + s * p.b_stride, p.xh + ((size_t)cur.kt * p.m_pad + m0) * 128, bytes, b_full + 8 * s);
        issued = i + 1;
        cur.advance(1, KT, TM);
      }
      for (int i = max(0, issued - SB); i < issued; i++) mbar_wait(b_full + 8 * (i % SB), (i / SB) & 1, 2u); // nothing in flight at exit
    }
  } else if (warp == MMA_WARP) {
    // ---- MMA issuer -------------------------------------------------------------------------------------
    if (lane == 0) {
      Cursor cur = start;
      bool alive = true, a_ready = false, b_ready = false;
      int i = 0, s = 0, sb = 0;
      uint32_t round = 0, bround = 0;
      for (int seg = 0; i < nsteps && alive; seg++) {
        const int len = min(KT - cur.kt, nsteps - i);
        const int buf = seg & 1, use = seg >> 1;
        if (use > 0) alive = mbar_wait(acc_empty + 8 * buf, (use - 1) & 1, 4u); // the drain of this buffer's previous segment
        if (!alive) break;
        tc_fence_after();
        const int64_t m0 = (int64_t)cur.tile_m * MAX_MT;
        const uint32_t idesc = idesc_f16((int)min((int64_t)MAX_MT, p.m_pad - m0));
        const uint32_t d = tmem_d + (uint32_t)(buf * MAX_MT);
        for (int j = 0; j < len && alive; j++, i++) {
          if (!a_ready) alive = mbar_wait(a_full + 8 * s, round & 1, 4u);
          if (alive && !b_ready) alive = mbar_wait(b_full + 8 * sb, bround & 1, 4u);
          if (!alive) break;
          tc_fence_after();
          const uint64_t adesc = smem_desc_sw128(a_ring + s * A_STAGE_BYTES);
          const uint64_t bdesc = smem_desc_sw128(b_ring + sb * p.b_stride);
          const int cs = s, csb = sb;
          if (++s == S) {
            s = 0;
            round++;
          }
          if (++sb == SB) {
            sb = 0;
            bround++;
          }
          // probe the next step's barriers now: the test's latency hides behind the issue of this step's MMAs
          a_ready = i + 1 < nsteps && mbar_try_wait(a_full + 8 * s, round & 1);
          b_ready = i + 1 < nsteps && mbar_try_wait(b_full + 8 * sb, bround & 1);
#pragma unroll
          for (int ks = 0; ks < BK / 16; ks++) umma_f16(d, adesc + (uint64_t)(ks * 2), bdesc + (uint64_t)(ks * 2), idesc, (j | ks) ? 1u : 0u);
          umma_commit(a_empty + 8 * cs);
          umma_commit(b_empty + 8 * csb);
        }
        if (alive) umma_commit(acc_full + 8 * buf);
        cur.advance(len, KT, TM);
      }
    }
  } else {
    // ---- drain: four warps, warp q reads accumulator lanes 32q.. (weight rows), all columns -----------------
    const int q = warp & 3; // tensor-memory lanes a warp may read are fixed by its index modulo 4
    const int half = (warp - EPI_WARP0) >> 2; // which half of the 32-column chunks this warp takes
    const int et = threadIdx.x - EPI_WARP0 * 32; // 0..127
    Cursor cur = start;
    bool alive = true;
    int i = 0;
    for (int seg = 0; i < nsteps && alive; seg++) {
      const int len = min(KT - cur.kt, nsteps - i);
      const bool whole = cur.kt == 0 && len == KT;
      const int buf = seg & 1, use = seg >> 1;
      const int tile_n = cur.tile_n, tile_m = cur.tile_m, tile = cur.tile(TM);
      const int64_t row = (int64_t)tile_n * TILE_N + 32 * q + lane;
      const int64_t m0 = (int64_t)tile_m * MAX_MT;
      const int mt = (int)min((int64_t)MAX_MT, p.m_pad - m0);
      // one thread waits for the accumulator and, for a tile shared with other CTAs, settles who stores and
      // who adds; the four warps then act on the same answers
      if (et == 0) {
        unsigned int t = mbar_wait_relaxed(acc_full + 8 * buf, use & 1, 8u) ? 0u : 0x80000000u;
        if (!whole && t == 0) {
          t = atomicAdd(p.tile_cnt + tile, 1u);
          if (t > 0) { // wait (bounded) until the first finisher's stores are visible
            const unsigned int *flag = p.tile_cnt + (size_t)p.tiles_n * p.tiles_m + tile;
            uint32_t spins = 0;
            unsigned int v = 0;
            do {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            } while (v == 0 && ++spins < WAIT_LIMIT);
            if (v == 0) {
              atomicOr(&g_prefill_status, 8u);
              t = 0x80000000u;
            }
          }
        }
        s_ticket = t;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
      const unsigned int ticket = s_ticket & 0x7fffffffu;
      alive = (s_ticket & 0x80000000u) == 0;
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory"); // s_ticket may be rewritten from here on
      if (alive) {
        tc_fence_after();
        const uint32_t lane_addr = tmem_d + (uint32_t)(buf * MAX_MT) + ((uint32_t)(32 * q) << 16);
        for (int c0 = 32 * half; c0 < mt; c0 += 32 * (EPI_WARPS / 4)) {
          uint32_t v[32];
          tmem_ld32(lane_addr + c0, v);
          const float ru_lane = (m0 + c0 + lane < p.m_pad) ? p.row_unscale[m0 + c0 + lane] : 0.f; // the chunk's 32 row factors
          tmem_ld_wait();
          const bool row_ok = row < p.w.n;
          if (p.y_dtype == XNQ_F32) {
            if (ticket == 0) drain_chunk<0>(v, ru_lane, p.y, p.ldy, row, m0 + c0, p.m, row_ok);
            else drain_chunk<1>(v, ru_lane, p.y, p.ldy, row, m0 + c0, p.m, row_ok);
          } else if (p.y_dtype == XNQ_F16) {
            drain_chunk<2>(v, ru_lane, p.y, p.ldy, row, m0 + c0, p.m, row_ok);
          } else {
            drain_chunk<3>(v, ru_lane, p.y, p.ldy, row, m0 + c0, p.m, row_ok);
          }
        }
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + 8 * buf); // this warp has read its lanes: the buffer may be overwritten
      if (!whole && alive) {
        if (ticket == 0) __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        if (ticket == 0 && et == 0) {
          unsigned int *flag = p.tile_cnt + (size_t)p.tiles_n * p.tiles_m + tile;
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(1u) : "memory");
        }
      }
      i += len;
      cur.advance(len, KT, TM);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == LOADER_WARP) tmem_dealloc(tmem_d, 2 * MAX_MT);
}

// ---- activation image -----------------------------------------------------------------------------------
// position of source element e (0..63) of a k-step inside the stored k-step, per weight format
__device__ __forceinline__ int kpos_q4_0(int e) { // stored chunk (b*4 + wi) holds [j, j+2, j+16, j+18, j+1, j+3, j+17, j+19] + 32b, j = 4wi
  const int b = e >> 5, x = e & 31, hi = x >> 4, y = x & 15, wi = y >> 2, t = y & 3;
  const int slot = (t & 1) * 4 + hi * 2 + (t >> 1);
  return (b * 4 + wi) * 8 + slot;
}
__device__ __forceinline__ int kpos_q4k(int e) { // stored chunk wi holds [l, l+2, 32+l, 32+l+2, l+1, l+3, 32+l+1, 32+l+3], l = 4wi
  const int hi = e >> 5, y = e & 31, wi = y >> 2, t = y & 3;
  const int slot = (t & 1) * 4 + hi * 2 + (t >> 1);
  return wi * 8 + slot;
}

// One CTA per activation row: Q8 quantize (the reference's activation blocks), dequantize, scale the row
// by a power of two so its largest magnitude lands in [2^11, 2^12), store fp16 into the swizzled image.
template <int ACT, typename XT>
__global__ void __launch_bounds__(256) prefill_prepare_acts(const XT *__restrict__ x, int64_t m, int64_t k, int64_t ldx, int64_t m_pad, int ksteps,
                                                            int wdtype, float wscale, uint8_t *__restrict__ xh, float *__restrict__ row_unscale,
                                                            unsigned int *__restrict__ tile_cnt, int tile_words) {
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  if (blockIdx.x == 0) // the persistent kernel's per-tile tickets and flags start every call at zero
    for (int i = threadIdx.x; i < tile_words; i += blockDim.x) tile_cnt[i] = 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t per_row = (int64_t)ksteps * 8; // 8-element groups in the padded row
  __half *img = reinterpret_cast<__half *>(xh);
  if (row >= m) { // padding rows: zeros
    for (int64_t t = threadIdx.x; t < per_row; t += blockDim.x) {
      const int64_t kt = t >> 3;
      *reinterpret_cast<uint4 *>(img + (kt * m_pad + row) * 64 + (t & 7) * 8) = make_uint4(0, 0, 0, 0);
    }
    if (threadIdx.x == 0) row_unscale[row] = 0.f;
    return;
  }
  const XT *xr = x + row * ldx;
  // pass 1: row maximum of the QUANTIZED-then-dequantized values is bounded by the raw maximum (codes <= 128/127 of it)
  float amax = 0.f;
  for (int64_t t = threadIdx.x; t < k / 8; t += blockDim.x) {
    float v[8];
    load8(xr + t * 8, v);
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
  // power of two s with amax * s in [2^10, 2^11): room for the 128/127 growth of the Q8_K codes
  int e = 0;
  if (amax > 0.f && amax < 3.0e38f) {
    (void)frexpf(amax, &e); // amax = f * 2^e, f in [0.5, 1)
  }
  const float rscale = amax > 0.f ? ldexpf(1.f, 11 - e) : 1.f;
  if (threadIdx.x == 0) row_unscale[row] = 1.f / (rscale * wscale); // exact: powers of two
  // pass 2: quantize per block, dequantize, scale, store. Whole warps stay together for the shuffles.
  const int64_t groups = k / 8;
  for (int64_t base = 0; base < per_row; base += blockDim.x) {
    const int64_t t = base + threadIdx.x;
    const bool valid = t < groups;
    float v[8];
    if (valid) load8(xr + t * 8, v);
    else {
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = 0.f;
    }
    const Quant8 q = ACT == XNQ_Q8_0 ? quantize8_q8_0(v, lane) : quantize8_q8k(v, lane);
    if (t >= per_row) continue;
    const float ds = q.d * rscale; // exact unless it leaves the normal range
    const int64_t kt = t >> 3;
    __half *dst = img + (kt * m_pad + row) * 64;
    const int sw = (int)(row & 7);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int code = (int)(int8_t)(((i < 4 ? q.lo : q.hi) >> (8 * (i & 3))) & 0xff);
      const int esrc = (int)((t & 7) * 8 + i);
      const int pos = wdtype == XNQ_Q4_0 ? kpos_q4_0(esrc) : (wdtype == XNQ_Q4K ? kpos_q4k(esrc) : esrc);
      const int chunk = pos >> 3;
      dst[((chunk ^ sw) << 3) + (pos & 7)] = __float2half_rn(valid ? (float)code * ds : 0.f);
    }
  }
}

int g_num_sms = 0;

template <typename RowT>
int launch_persistent_fmt(const PrefillArgs &a, unsigned ctas, size_t smem, cudaStream_t s) {
  prefill_persistent_kernel<RowT><<<ctas, NTHREADS_SK, smem, s>>>(a);
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

constexpr size_t PREFILL_SMEM = 226 * 1024; // everything an SM offers minus the static barriers and a reserve

} // namespace

static size_t tile_words(int64_t m_pad, int64_t n) { // tickets + flags of the persistent kernel
  const size_t tiles = (size_t)((n + TILE_N - 1) / TILE_N) * (size_t)((m_pad + MAX_MT - 1) / MAX_MT);
  return (2 * tiles * 4 + 255) & ~(size_t)255;
}

size_t prefill_workspace_bytes(int64_t m, int64_t k, int64_t n) {
  const int64_t m_pad = (m + 15) / 16 * 16;
  const int64_t ksteps = (k + BK - 1) / BK;
  return (size_t)ksteps * m_pad * 128 + (((size_t)m_pad * 4 + 255) & ~(size_t)255) + tile_words(m_pad, n) + 256;
}

int launch_prefill(const WeightView &w, float wscale, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy,
                   void *workspace, cudaStream_t s) {
  const int64_t k = w.k;
  const int64_t m_pad = (m + 15) / 16 * 16;
  const int ksteps = (int)((k + BK - 1) / BK);
  float *row_unscale = static_cast<float *>(workspace);
  unsigned int *tile_cnt = reinterpret_cast<unsigned int *>(static_cast<uint8_t *>(workspace) + ((((size_t)m_pad * 4 + 255) & ~(size_t)255)));
  const size_t cnt_bytes = tile_words(m_pad, w.n);
  uint8_t *xh = reinterpret_cast<uint8_t *>(tile_cnt) + cnt_bytes;
  const int act = act_dtype_for(w.dtype);
#define XNQ_PREP(ACT, XT)                                                                                                   \
  prefill_prepare_acts<ACT, XT><<<(unsigned)m_pad, 256, 0, s>>>(static_cast<const XT *>(x), m, k, ldx, m_pad, ksteps, w.dtype, wscale, xh, \
                                                                row_unscale, tile_cnt, (int)(cnt_bytes / 4))
  if (act == XNQ_Q8_0) {
    if (x_dtype == XNQ_F32) XNQ_PREP(XNQ_Q8_0, float);
    else if (x_dtype == XNQ_F16) XNQ_PREP(XNQ_Q8_0, __half);
    else XNQ_PREP(XNQ_Q8_0, __nv_bfloat16);
  } else {
    if (x_dtype == XNQ_F32) XNQ_PREP(XNQ_Q8K, float);
    else if (x_dtype == XNQ_F16) XNQ_PREP(XNQ_Q8K, __half);
    else XNQ_PREP(XNQ_Q8K, __nv_bfloat16);
  }
#undef XNQ_PREP
  XNQ_CUDA(cudaGetLastError());
  count_launch();

  PrefillArgs a{};
  a.w = w;
  a.xh = xh;
  a.row_unscale = row_unscale;
  a.y = y;
  a.y_dtype = y_dtype;
  a.ldy = ldy;
  a.m = m;
  a.m_pad = m_pad;
  a.ksteps = ksteps;
  a.nstages = NSTAGES;
  // shared-memory plan: A ring | B ring (as deep as fits, at most 8) | raw rings
  const int slot = w.dtype == XNQ_Q6K ? 80 : 48;
  const uint32_t mt_max = (uint32_t)std::min<int64_t>(MAX_MT, m_pad);
  a.b_stride = (mt_max * 128 + 1023) & ~1023u;
  const size_t raw_bytes = (size_t)RAW_DEPTH * PRODUCERS * slot;
  const size_t fixed = (size_t)NSTAGES * A_STAGE_BYTES + raw_bytes + 1024; // + alignment slack
  a.b_stages = (int)std::min<size_t>(8, (PREFILL_SMEM - fixed) / a.b_stride);
  if (a.b_stages < 2) return fail(XNQ_ERR_SIZE, "prefill: shared-memory plan does not fit");
  a.b_off = NSTAGES * A_STAGE_BYTES;
  a.raw_off = a.b_off + a.b_stages * a.b_stride;
  a.wscale = wscale;
  const dim3 grid((unsigned)((w.n + TILE_N - 1) / TILE_N), (unsigned)((m_pad + MAX_MT - 1) / MAX_MT));
  a.tiles_n = (int)grid.x;
  a.tiles_m = (int)grid.y;
  a.units = (long long)grid.x * grid.y * ksteps;
  a.whole_tiles = y_dtype == XNQ_F32 ? 0 : 1;
  a.tile_cnt = tile_cnt;
  profile_mark(s, true);
  int rc;
  const long long tiles = (long long)grid.x * grid.y;
  const long long want = a.whole_tiles ? tiles : std::max<long long>(1, a.units / 8); // at least 8 k-steps per CTA
  const unsigned ctas = (unsigned)std::min<long long>(g_num_sms, want);
  switch (w.dtype) {
    case XNQ_Q4_0: rc = launch_persistent_fmt<RowQ4_0>(a, ctas, PREFILL_SMEM, s); break;
    case XNQ_Q8_0: rc = launch_persistent_fmt<RowQ8_0>(a, ctas, PREFILL_SMEM, s); break;
    case XNQ_Q4K: rc = launch_persistent_fmt<RowQ4K>(a, ctas, PREFILL_SMEM, s); break;
    case XNQ_Q6K: rc = launch_persistent_fmt<RowQ6K>(a, ctas, PREFILL_SMEM, s); break;
    default: rc = fail(XNQ_ERR_DTYPE, "prefill: dtype %d", w.dtype);
  }
  profile_mark(s, false);
  return rc;
}

int prefill_init(int device) {
  cudaDeviceProp prop;
  XNQ_CUDA(cudaGetDeviceProperties(&prop, device));
  g_num_sms = prop.multiProcessorCount;
  XNQ_CUDA(cudaFuncSetAttribute(prefill_persistent_kernel<RowQ4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREFILL_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(prefill_persistent_kernel<RowQ8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREFILL_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(prefill_persistent_kernel<RowQ4K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREFILL_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(prefill_persistent_kernel<RowQ6K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREFILL_SMEM));
  unsigned int zero = 0;
  XNQ_CUDA(cudaMemcpyToSymbol(g_prefill_status, &zero, sizeof(zero)));
  return XNQ_OK;
}

int prefill_status(unsigned int *bits) {
  XNQ_CUDA(cudaMemcpyFromSymbol(bits, g_prefill_status, sizeof(*bits)));
  return XNQ_OK;
}

} // namespace xnq
