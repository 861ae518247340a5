// Small batches (2 <= m <= 64 activation rows per pass) on the 5th-generation tensor cores with exact
// integer arithmetic: tcgen05.mma.kind::i8, one tensor-memory accumulator slice per 32-element block.
//
// The reference's dots are exact integer sums over one 32-element (sub-)block, scaled in f32
// (k_quants.rs:287-304 Q4_0, 677-691 Q8_0, 1337-1416 Q4_K). One MMA
//
//     D[128 weight rows, NP activation rows] = A[128, 32] . B[NP, 32]^T          (s8 x s8 -> s32, no accumulation)
//
// is exactly those sums for 128 x NP (weight row, activation row) pairs and one block, so every MMA writes
// its own slice of tensor memory and the drain warps apply the block's scales to it in f32 exactly as the
// CPU code does: integer sub-block scales and mins for Q4_K (min term from the activations' 32-sums with
// dp4a), f16 block scale times f16-rounded activation scale for Q4_0 / Q8_0. Nothing is rounded before the
// f32 scaling, so results stay within the f32-accumulate bound (2e-3) at every batch size served.
//
// Roles of the 27 warps of a CTA (one CTA per SM, persistent):
//   producer (1)    one thread requests, per 256-k step, the 1-D bulk copies of the quantized activations (already in
//                   the MMA's shared-memory layout) and of their per-block metadata into rings of stages guarded by
//                   mbarriers; when the kernel starts it also asks for the CTA's share of the weight's bytes to be
//                   brought into L2 in long contiguous runs.
//   converters (8)  two groups of four warps, one thread per weight row; the groups take alternate 256-k steps, so a step's
//                   chain of waits, loads, stores and fences has two steps' time to run in. Every warp fetches the code bytes of its own 32 rows itself, several steps ahead, with
//                   16-byte cp.async copies into a ring of warp-private slots (consecutive lanes take consecutive
//                   16 bytes of a row, so the requests are whole sectors; nothing but the warp's own
//                   cp.async.wait_group and __syncwarp orders them), unpacks 4-bit codes to int8 (or copies int8
//                   codes) into the 128-byte-swizzled K-major operand image the MMA reads, and hands the rows' scale
//                   bytes on to the drain. (Tiled TMA boxes of 128 rows x 144..256 bytes were tried first:
//                   a box took 5000 to 7000 cycles to arrive, with or without the bytes in L2, about 17 cycles per box
//                   row, which held the whole kernel at a third of the memory's rate. One bulk copy per row before
//                   that: the copy engine takes some 60 ns per copy whatever its size.)
//   MMA issuers (2) one thread per half step issues its four K = 32 MMAs into accumulator buffer h and commits them; an
//                   MMA of this shape keeps its issuing thread busy for about 134 cycles whatever M (64 / 128) and
//                   N <= 128 are, while two issuing threads reach twice the rate (measured), so the halves of a step
//                   are issued by two warps;
//   drain (16)      two groups of eight warps; group h owns accumulator buffer h: reads its slices back with
//                   tcgen05.ld, scales, and keeps f32 sums in registers across the k steps of a tile; two warps
//                   per accumulator lane quarter split the columns. At the end of a segment the odd half steps'
//                   sums are added to the even ones' (always in that order).
//
// Work is the flattened (tile of 128 weight rows, 256-k step) space, cut into equal contiguous ranges, one
// per CTA, so all SMs finish together however few tiles there are. A tile whose steps are split between
// CTAs is summed deterministically: every part is written to a scratch slot, an arrival ticket elects the
// last part, and that CTA adds the parts in k order and stores y.
//
// Every wait is bounded; on expiry a status bit is set and the roles fall through to the common exit, where
// tensor memory is released.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "xnq_common.cuh"
#include "xnq_quantize_act.cuh"

namespace xnq {

__device__ unsigned int g_imma_status; // sticky: 1 producer, 2 converter, 4 mma, 8 drain wait expired
#ifdef XNQ_DEV_TRACE
__device__ long long g_imma_trace[32]; // development builds only: cycles block 0's roles spend in each wait
__device__ long long g_imma_tl[8 * 64];  // development builds only: block 0's per-unit time line (clock64), 8 points x 64 units
#define XNQ_TL(pt, i) do { if (blockIdx.x == 0 && (i) < 64) g_imma_tl[(pt) * 64 + (i)] = clock64(); } while (0)
#define XNQ_GT(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) { unsigned long long g_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_)); g_imma_trace[i] = (long long)g_; } } while (0)
#define XNQ_TACC(i) do { const long long t1_ = clock64(); tacc[i] += t1_ - t0_; t0_ = t1_; } while (0)
#define XNQ_TDECL long long tacc[6] = {0, 0, 0, 0, 0, 0}; long long t0_ = clock64()
#define XNQ_TDUMP(base, cond) do { if ((cond) && blockIdx.x == 0) for (int i_ = 0; i_ < 6; i_++) g_imma_trace[(base) + i_] = tacc[i_]; } while (0)
#else
#define XNQ_GT(i) do { } while (0)
#define XNQ_TL(pt, i) do { } while (0)
#define XNQ_TACC(i) do { } while (0)
#define XNQ_TDECL do { } while (0)
#define XNQ_TDUMP(base, cond) do { } while (0)
#endif

namespace {

constexpr int TILE_N = 128;         // weight rows per tile = UMMA M
constexpr int MAX_NP = 64;          // activation rows per pass = UMMA N (multiple of 16)
constexpr int CONV_WARPS = 8, DRAIN_WARPS = 16;
constexpr int ACT_PRODUCER_WARP = 0, MMA_WARP = 1, CONV_WARP0 = 3, DRAIN_WARP0 = CONV_WARP0 + CONV_WARPS; // MMA issuers: warps 1 and 2
constexpr int NTHREADS = (DRAIN_WARP0 + DRAIN_WARPS) * 32; // 864
constexpr int A_STAGE_BYTES = TILE_N * 128; // one 128-k half step of int8 codes
constexpr int MAX_A_STAGES = 8, SIDE_STAGES = 8, MAX_RAW_STAGES = 8; // side stages are small (scale bytes and records of one step): enough of them that
                                                                   // the converters, which fill them, never wait for the drain, which frees them
constexpr int HDR_BYTES = TILE_N * 16;      // per 256-k step: 16 bytes of scale data per weight row
constexpr int TMEM_COLS = 512;              // all of the SM's tensor memory: 512 / (4 slices x NP) accumulator buffers, at most 8
constexpr size_t IMMA_SMEM = 226 * 1024;
constexpr uint32_t PF_CHUNK = 16384;              // bytes per L2 prefetch request
constexpr size_t PF_MAX_BYTES = 80ull << 20;      // larger weights are not prefetched whole: they would push each other out of L2

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
// One wait attempt: the thread is suspended by the hardware until the phase completes or a system-chosen time limit
// passes (it takes no issue slots meanwhile, unlike a test_wait spin, which with two dozen polling warps per SM slowed
// the threads that issue copies and MMAs several times over).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// the same with a suspend-time hint in nanoseconds: the hardware may keep the thread suspended that long before it
// returns false (a plain try_wait returned after a system-chosen, short time, and two dozen waiting warps per SM then
// spent a large share of the SM's issue slots re-issuing their waits: 60 % issue utilisation, a fifth of it in the
// unit that executes barrier instructions)
__device__ __forceinline__ bool mbar_test_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long wall_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull; // a wait that lasts two seconds is given up
// bounded wait of one thread
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int bit) {
  if (mbar_test(bar, parity)) return true;
  unsigned long long t0 = 0;
  for (unsigned int attempt = 1;; attempt++) { // the wall clock is read on every 16th failed attempt only
    if (mbar_test_hint(bar, parity, 1000000u)) return true;
    if ((attempt & 15u) == 0) {
      const unsigned long long now = wall_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) break;
    }
  }
  atomicOr(&g_imma_status, bit);
  return false;
}
// bounded wait of a whole warp: lane 0 polls (32 lanes polling one word keep the shared-memory pipe busy for
// nothing), the other lanes park on the warp barrier
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, unsigned int bit) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, bit) ? 1 : 0;
  __syncwarp();
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
// asks for a run of global memory to be brought into L2 (a hint; nothing waits for it)
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// 16-byte asynchronous copy global -> shared, bypassing L1; src_bytes 0 writes zeros instead (the address is not read)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most `pending` of this thread's committed groups are still in flight
__device__ __forceinline__ void cp_async_wait(int pending) {
  switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
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
// D = A . B^T (no accumulation: every MMA owns its accumulator slice)
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u)
      : "memory");
}
// arrives on the mbarrier once every MMA issued so far by this thread has finished reading smem / writing tmem
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tmem_ld<4>(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
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
// kind::i8 instruction descriptor: D s32 (2 at [4,6)), A and B signed 8-bit (1 at [7,10) / [10,13)), both K-major,
// N >> 3 at [17,23), M >> 4 at [24,29).
__device__ __forceinline__ uint32_t idesc_i8(int umma_n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

struct ImmaArgs {
  WeightView w;
  const uint8_t *bimg; // quantized activations in operand layout: [half steps][NP rows x 128 bytes, 128-byte swizzle]
  const uint8_t *meta; // per 256-k step and activation row: 32 bytes of scales / sums (layout per format below)
  void *y;
  int y_dtype;
  int64_t ldy;
  int64_t m;           // activation rows of this pass (<= NP)
  int nsteps;          // 256-k steps per tile
  int tiles;
  int units;           // tiles * nsteps
  int units_q, units_r; // CTA c works on units [c * units_q + min(c, units_r), + units_q + (c < units_r)): set at launch, so that
                        // no thread divides 64-bit numbers before its first copy
  unsigned int *tile_cnt; // [tiles] arrival tickets of split tiles, zeroed by the prepare kernel
  float *partials;        // [2 * grid][NP][128] partial sums of split tiles
  float *pair_scratch;    // [grid][NP][128]: the odd half steps' sums on their way to the even ones'
  // raw weight bytes: stream 0 holds the codes (Q4_K: the whole 144-byte super-blocks), stream 1 the f16 block scales of Q4_0 / Q8_0
  const uint8_t *src[2];
  int nstreams;
  uint32_t row_bytes[2];  // bytes of one weight row in the stream
  uint32_t step_bytes[2]; // bytes of one 256-k step of a row
  uint32_t code_off;      // where the codes start inside a step of stream 0 (Q4_K: after the 16 header bytes)
  // each CTA asks for its share of every stream (whole, contiguous rows) to be brought into L2 when it starts
  const uint8_t *pf_base[2];
  unsigned long long pf_bytes[2], pf_share[2]; // share: a multiple of PF_CHUNK; bytes 0: no prefetch
  int raw_stages, b_stages, a_stages;
  uint32_t raw_stage_bytes, b_stage_bytes, side_stage_bytes;
  uint32_t a_off, b_off, raw_off0, side_off; // offsets from the 1024-aligned base of dynamic shared memory; a raw stage holds eight warp slots
};

// the flattened (tile, step) space is cut into contiguous ranges: the first units_r CTAs take units_q + 1 units, the others units_q
__device__ __forceinline__ int cta_first_unit(int c, int q, int r) { return c * q + min(c, r); }
__device__ __forceinline__ int cta_of(int u, int q, int r) {
  const int big = r * (q + 1); // units held by the CTAs that take q + 1
  return u < big ? u / (q + 1) : r + (u - big) / q;
}

// ---- converters: raw bytes of (row, 64 of the step's 256 k) -> 64 bytes of int8 codes ------------------------
// A warp slot holds the step's code bytes of the warp's 32 rows, STEP bytes per row; the 16-byte chunk c of row r sits
// at r * STEP + ((c ^ (r & (STEP / 16 - 1))) << 4), so that 32 lanes reading chunk c of their own rows touch all the
// banks. row: shared address of the lane's row in the slot; key: the lane's row number in the slot; h: half step;
// p: which 64 k of the half step.
template <int STEP>
__device__ __forceinline__ uint4 raw_chunk(uint32_t row, int key, int c) {
  return lds128(row + (uint32_t)((c ^ (key & (STEP / 16 - 1))) << 4));
}
struct ConvQ8_0 { // 256 code bytes per row and step
  static constexpr int STEP = 256;
  __device__ static __forceinline__ void run(uint32_t row, int key, int h, int p, uint4 (&out)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) out[i] = raw_chunk<STEP>(row, key, 8 * h + 4 * p + i);
  }
};
__device__ __forceinline__ uint32_t nib_lo_s8(uint32_t w) { return (((w & 0x0f0f0f0fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u; } // code - 8 per byte
__device__ __forceinline__ uint32_t nib_hi_s8(uint32_t w) { return ((((w >> 4) & 0x0f0f0f0fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }
struct ConvQ4_0 { // eight blocks of 16 nibble bytes per row and step; element j < 16 low nibble of byte j, j >= 16 high nibble of byte j - 16
  static constexpr int STEP = 128;
  __device__ static __forceinline__ void run(uint32_t row, int key, int h, int p, uint4 (&out)[4]) {
#pragma unroll
    for (int bb = 0; bb < 2; bb++) {
      const uint4 q = raw_chunk<STEP>(row, key, 4 * h + 2 * p + bb);
      out[2 * bb] = make_uint4(nib_lo_s8(q.x), nib_lo_s8(q.y), nib_lo_s8(q.z), nib_lo_s8(q.w));
      out[2 * bb + 1] = make_uint4(nib_hi_s8(q.x), nib_hi_s8(q.y), nib_hi_s8(q.z), nib_hi_s8(q.w));
    }
  }
};
struct ConvQ4K { // 128 code bytes per row and step: four 32-byte chunks; chunk c = sub-block 2c in the low nibbles, 2c+1 in the high ones
  static constexpr int STEP = 128;
  __device__ static __forceinline__ void run(uint32_t row, int key, int h, int p, uint4 (&out)[4]) {
    const uint4 a = raw_chunk<STEP>(row, key, 2 * (2 * h + p)), b = raw_chunk<STEP>(row, key, 2 * (2 * h + p) + 1);
    out[0] = make_uint4(a.x & 0x0f0f0f0fu, a.y & 0x0f0f0f0fu, a.z & 0x0f0f0f0fu, a.w & 0x0f0f0f0fu);
    out[1] = make_uint4(b.x & 0x0f0f0f0fu, b.y & 0x0f0f0f0fu, b.z & 0x0f0f0f0fu, b.w & 0x0f0f0f0fu);
    out[2] = make_uint4((a.x >> 4) & 0x0f0f0f0fu, (a.y >> 4) & 0x0f0f0f0fu, (a.z >> 4) & 0x0f0f0f0fu, (a.w >> 4) & 0x0f0f0f0fu);
    out[3] = make_uint4((b.x >> 4) & 0x0f0f0f0fu, (b.y >> 4) & 0x0f0f0f0fu, (b.z >> 4) & 0x0f0f0f0fu, (b.w >> 4) & 0x0f0f0f0fu);
  }
};

// ---- drain: scale the four slices of a half step and add them to the running sums ----------------------------
// hdr: the row's 16 scale bytes of the 256-k step; meta: shared address of the step's per-activation-row records
// (32 bytes each); v[j][c]: slice j (block 4h + j of the step), column c of this thread; c0: first column.
//   Q4_0 / Q8_0  hdr = eight f16 block scales; record = eight f32 activation block scales
//   Q4_K         hdr = f16 d, f16 dmin, four 24-bit fields sc[2g] | sc[2g+1] << 6 | mn[2g] << 12 | mn[2g+1] << 18;
//                record = {lo(h=0), hi(h=0), lo(h=1), hi(h=1), f32 d, 0, 0, 0}: the four sub-blocks' 32-sums of the
//                activation codes, s = 128 * hi + lo with lo in 0..127 (one byte each)
template <int CH>
struct DrainBlockScaled {
  __device__ static __forceinline__ void run(const uint4 &hdr, uint32_t meta, int h, int c0, const uint32_t (&v)[4][CH], float *acc) {
    const uint32_t w0 = h ? hdr.z : hdr.x, w1 = h ? hdr.w : hdr.y;
    const __half2 h0 = *reinterpret_cast<const __half2 *>(&w0), h1 = *reinterpret_cast<const __half2 *>(&w1);
    const float dw[4] = {__low2float(h0), __high2float(h0), __low2float(h1), __high2float(h1)};
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const uint4 da = lds128(meta + (uint32_t)(c0 + c) * 32 + 16 * h);
      acc[c] += (float)(int)v[0][c] * (dw[0] * __uint_as_float(da.x));
      acc[c] += (float)(int)v[1][c] * (dw[1] * __uint_as_float(da.y));
      acc[c] += (float)(int)v[2][c] * (dw[2] * __uint_as_float(da.z));
      acc[c] += (float)(int)v[3][c] * (dw[3] * __uint_as_float(da.w));
    }
  }
};
template <int CH>
struct DrainQ4K {
  __device__ static __forceinline__ void run(const uint4 &hdr, uint32_t meta, int h, int c0, const uint32_t (&v)[4][CH], float *acc) {
    const __half2 dm = *reinterpret_cast<const __half2 *>(&hdr.x);
    const float d = __low2float(dm), dmin = __high2float(dm);
    // fields 2h and 2h + 1: bits [48h, 48h + 48) of the 96-bit field array in hdr.y, hdr.z, hdr.w
    const uint32_t lo32 = h ? __funnelshift_r(hdr.z, hdr.w, 16) : hdr.y;
    const uint32_t hi16 = h ? (hdr.w >> 16) : (hdr.z & 0xffffu);
    const uint32_t f0 = lo32 & 0xffffffu, f1 = __funnelshift_r(lo32, hi16, 24) & 0xffffffu;
    const int sc0 = f0 & 63, sc1 = (f0 >> 6) & 63, sc2 = f1 & 63, sc3 = (f1 >> 6) & 63;
    const uint32_t mins = ((f0 >> 12) & 63) | (((f0 >> 18) & 63) << 8) | (((f1 >> 12) & 63) << 16) | (((f1 >> 18) & 63) << 24);
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const uint32_t rec = meta + (uint32_t)(c0 + c) * 32;
      const uint2 bs = lds64(rec + 8 * h);
      const float da = __uint_as_float(lds32(rec + 16));
      const int isum = sc0 * (int)v[0][c] + sc1 * (int)v[1][c] + sc2 * (int)v[2][c] + sc3 * (int)v[3][c];
      const int msum = dp4a_uu(mins, bs.x, 0) + dp4a_us(mins, bs.y, 0) * 128;
      acc[c] += da * (d * (float)isum - dmin * (float)msum);
    }
  }
};

template <typename Conv, template <int> class Drain, int NP>
__global__ void __launch_bounds__(NTHREADS, 1) imma_kernel(const __grid_constant__ ImmaArgs p) {
  // Drain warps per half-step group: eight, two per accumulator lane quarter, splitting the columns. (Four per group with 16
  // activation rows, which halves the fixed cost per step, was no faster: each warp's chain of loads from tensor memory and
  // arithmetic per half step then takes longer than the MMAs of a step.)
  constexpr int DWG = 8;
  constexpr int NPT = NP / (DWG / 4); // columns per drain thread
  constexpr int CH = NPT > 16 ? 4 : (NPT > 8 ? 8 : NPT); // columns read back at a time: what the register budget holds next to the sums
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u; // operand stages need 1024-byte alignment
  constexpr int NBUF = TMEM_COLS / (4 * NP) > 8 ? 8 : TMEM_COLS / (4 * NP); // accumulator buffers (even: buffer parity = half step parity)
  constexpr int BUF_COLS = 4 * NP;
  // barriers: b_full [4], side_full/side_empty [8], a_full/mma_done [8], acc_empty [8]
  __shared__ __align__(8) uint64_t bars[44];
  __shared__ uint32_t tmem_slot;
  __shared__ unsigned int s_ticket;
  const uint32_t b_full = smem_u32(bars), side_full = b_full + 32, side_empty = b_full + 96, a_full = b_full + 160, mma_done = b_full + 224,
                 acc_empty = b_full + 288;
  XNQ_GT(26);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int RS = p.raw_stages, BS = p.b_stages, AS = p.a_stages;
  const int NB = min(NBUF, AS); // accumulator buffers in use: a drain group waiting on mma_done must not be lapped by the MMA thread,
                                // which can run ahead by NB half steps, so the ring of mma_done barriers (AS) is at least that long
  const int KT = p.nsteps;
  const int u0 = cta_first_unit((int)blockIdx.x, p.units_q, p.units_r);
  const int nunits = p.units_q + ((int)blockIdx.x < p.units_r ? 1 : 0);
  const int tile0 = u0 / KT, kt0 = u0 - tile0 * KT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; s++) {
      mbar_init(a_full + 8 * s, CONV_WARPS / 2); // the four converter warps of the step's group (one barrier per step: entries 0 .. BS - 1)
      mbar_init(mma_done + 8 * s, 1);            // the half step's MMAs have read their operands and written their slices
      mbar_init(acc_empty + 8 * s, DWG);
      mbar_init(side_full + 8 * s, 1 + CONV_WARPS / 2); // the producer's transaction + the four converter warps that copy the scale bytes
      mbar_init(side_empty + 8 * s, 2 * DWG);
    }
    for (int s = 0; s < 4; s++) mbar_init(b_full + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) { // one warp owns the tensor-memory allocation
    tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents(); // the next kernel in the stream may be set up while this one runs
  const uint32_t tmem_d = tmem_slot;

  if (warp == ACT_PRODUCER_WARP) {
    // ---- activation producer: per 256-k step the activations' operand image and their records ----
    if (lane == 0) {
      // A 256-k step of a tile is 128 separate runs of 144 to 256 bytes, 2 to 4 KB apart. So that DRAM is read in long
      // contiguous runs all the same, the weight is asked into L2 whole when the kernel starts, every CTA asking for its
      // share of the bytes (not of the work: any CTA's copies then hit in L2, or go to DRAM when they are early).
      for (int st = 0; st < p.nstreams; st++) {
        const unsigned long long o0 = p.pf_share[st] * blockIdx.x, o1 = min(o0 + p.pf_share[st], p.pf_bytes[st]);
        for (unsigned long long o = o0; o < o1; o += PF_CHUNK) bulk_prefetch_l2(p.pf_base[st] + o, (uint32_t)min((unsigned long long)PF_CHUNK, o1 - o));
      }
      pdl_wait();
      bool alive = true;
      int kt = kt0, bs = 0;
      uint32_t b_ph = 0; // (i / BS) & 1
      for (int i = 0; i < nunits && alive; i++) {
        const int ss = i % SIDE_STAGES;
        // the B stage of step i - BS is free once that step's second half has been multiplied: BS = AS / 2, so this is
        // the barrier of half step 2 i + 1 one phase back (a second commit per step cost the issuing thread over a
        // thousand cycles)
        if (i >= BS) alive = mbar_wait(mma_done + 8 * (2 * bs), b_ph ^ 1u, 1u) && mbar_wait(mma_done + 8 * (2 * bs + 1), b_ph ^ 1u, 1u);
        if (alive && i >= SIDE_STAGES) alive = mbar_wait(side_empty + 8 * ss, ((i / SIDE_STAGES) - 1) & 1, 1u);
        if (!alive) break;
        mbar_expect_tx(b_full + 8 * bs, p.b_stage_bytes);
        mbar_expect_tx(side_full + 8 * ss, (uint32_t)NP * 32u);
        bulk_g2s(base + p.b_off + bs * p.b_stage_bytes, p.bimg + ((size_t)kt * 2) * (NP * 128), p.b_stage_bytes, b_full + 8 * bs);
        bulk_g2s(base + p.side_off + ss * p.side_stage_bytes + HDR_BYTES, p.meta + (size_t)kt * (NP * 32), (uint32_t)NP * 32u, side_full + 8 * ss);
        XNQ_TL(1, i);
        if (++kt == KT) kt = 0;
        if (++bs == BS) bs = 0, b_ph ^= 1u;
      }
    }
  } else if (warp == MMA_WARP || warp == MMA_WARP + 1) {
    // ---- MMA issuers: one thread per half step. A tcgen05.mma of this shape keeps the thread that issues it busy for about
    // 134 cycles, but two threads issuing into different accumulator slices get twice the rate (measured up to N = 64), so
    // the two halves of a step are issued by two warps, each with its own commit. ----
    const int hh = warp - MMA_WARP;
    if (lane == 0) {
      const uint32_t idesc = idesc_i8(NP);
      bool alive = true;
      XNQ_TDECL;
      int bs = 0, nb = 0; // i % BS, i % (NB / 2): AS and NB are even, so half step j = 2 i + h uses A stage 2 bs + h and buffer 2 nb + h
      uint32_t b_ph = 0, acc_ph = 0; // (i / BS) & 1 = (j / AS) & 1, (j / NB) & 1
      for (int i = 0; i < nunits && alive; i++) {
        XNQ_TACC(0);
        alive = mbar_wait(b_full + 8 * bs, b_ph, 4u);
        XNQ_TACC(1);
        if (alive) alive = mbar_wait(a_full + 8 * bs, b_ph, 4u); // both halves of the step's operand image
        XNQ_TACC(2);
        {
          const int h = hh;
          const int sa = 2 * bs + h, buf = 2 * nb + h;
          XNQ_TACC(0);
          if (alive && 2 * i >= NB) alive = mbar_wait(acc_empty + 8 * buf, acc_ph ^ 1u, 4u); // the drain of the buffer's previous half step
          XNQ_TACC(3);
          if (!alive) break;
          if (h == 0) XNQ_TL(4, i);
          tc_fence_after();
          const uint64_t adesc = smem_desc_sw128(base + p.a_off + sa * A_STAGE_BYTES);
          const uint64_t bdesc = smem_desc_sw128(base + p.b_off + bs * p.b_stage_bytes + h * (NP * 128));
#pragma unroll
          for (int q = 0; q < 4; q++) // K = 32 per instruction: advance 32 bytes inside the swizzle row; slice q of the buffer
            umma_i8(tmem_d + (uint32_t)(buf * BUF_COLS + q * NP), adesc + (uint64_t)(q * 2), bdesc + (uint64_t)(q * 2), idesc);
          XNQ_TACC(4);
          // the arrival serves the drain (the slices are written) and, together with the other half's, the converters and the
          // activation producer (the stages are free)
          umma_commit(mma_done + 8 * sa);
          XNQ_TACC(5);
          if (h == 1) XNQ_TL(5, i);
        }
        if (++bs == BS) bs = 0, b_ph ^= 1u;
        if (2 * ++nb == NB) nb = 0, acc_ph ^= 1u;
      }
      XNQ_TDUMP(6, hh == 0);
    }
  } else if (warp < DRAIN_WARP0) {
    // ---- converters: group g (four warps, one thread per weight row) produces the steps i = g, g + 2, ... of this CTA: a
    // step's chain of waits, loads, stores and fences has the time of two steps' MMAs to run in ----
    constexpr int STEP = Conv::STEP, CPR = STEP / 16, RPI = 32 / CPR; // code bytes per row and step; 16-byte chunks per row; rows per copy instruction
    constexpr uint32_t SLOT = 32 * STEP + 512;                          // a warp's slot: its rows' code bytes, then 16 scale bytes per row
    const int cw = warp - CONV_WARP0;
    const int r0 = (cw & 3) * 32, r = r0 + lane, g = cw >> 2;
    const int sw = r & 7;
    const int D = RS >> 1; // slots per warp: RS steps are in flight per CTA, half of them this group's
    const uint32_t slot0 = base + p.raw_off0 + (uint32_t)(cw * D) * SLOT;
    const int64_t n = p.w.n;
    // the warp's own loads, D of its steps ahead: lane l copies chunk l % CPR of row q * RPI + l / CPR in instruction q
    int l_i = g, l_tile = tile0, l_kt = kt0 + g, l_s = 0;
    while (l_kt >= KT) l_kt -= KT, l_tile++;
    auto issue = [&]() {
      const uint32_t dst = slot0 + (uint32_t)l_s * SLOT;
      const int c = lane % CPR;
      const uint32_t in_row = (uint32_t)l_kt * p.step_bytes[0] + p.code_off + (uint32_t)(c * 16); // a row's bytes end at a multiple of 16
      const uint32_t bytes = in_row + 16 <= p.row_bytes[0] ? 16u : 0u;
#pragma unroll
      for (int q = 0; q < CPR; q++) {
        const int rw = q * RPI + lane / CPR;
        const int64_t grow = (int64_t)l_tile * TILE_N + r0 + rw;
        const bool ok = grow < n;
        cp_async16(dst + (uint32_t)(rw * STEP + ((c ^ (rw & (CPR - 1))) << 4)), p.src[0] + (size_t)(ok ? grow : n - 1) * p.row_bytes[0] + in_row, ok ? bytes : 0u);
      }
      { // the rows' 16 scale bytes of the step: the head of the Q4_K super-block, or eight f16 block scales
        const int st = p.nstreams - 1;
        const int64_t grow = (int64_t)l_tile * TILE_N + r;
        const bool ok = grow < n && (uint32_t)l_kt * p.step_bytes[st] + 16 <= p.row_bytes[st];
        cp_async16(dst + 32 * STEP + lane * 16, p.src[st] + (size_t)(grow < n ? grow : n - 1) * p.row_bytes[st] + (ok ? (size_t)l_kt * p.step_bytes[st] : 0), ok ? 16u : 0u);
      }
      l_i += 2, l_kt += 2;
      while (l_kt >= KT) l_kt -= KT, l_tile++;
      if (++l_s == D) l_s = 0;
    };
    for (int u = 0; u < D; u++) { // weights are immutable after upload: nothing here waits for the kernel that prepares the activations
      if (l_i < nunits) issue();
      cp_async_commit();
    }
    bool alive = true;
    XNQ_TDECL;
    int rs = 0, bs = g % BS;
    uint32_t a_ph = (uint32_t)(g / BS) & 1u; // (i / BS) & 1
    for (int i = g; i < nunits && alive; i += 2) {
      const int ss = i % SIDE_STAGES;
      XNQ_TACC(0);
      cp_async_wait(D - 1); // one group per step and lane, committed in step order: step i's has landed
      __syncwarp();         // ... for every lane of the warp
      XNQ_TACC(1);
      if (threadIdx.x == CONV_WARP0 * 32) XNQ_TL(2, i);
      const uint32_t slot = slot0 + (uint32_t)rs * SLOT;
      { // hand the row's 16 scale bytes to the drain
        if (i >= SIDE_STAGES) alive = mbar_wait_warp(side_empty + 8 * ss, ((i / SIDE_STAGES) - 1) & 1, 2u);
        XNQ_TACC(2);
        if (!alive) break;
        const uint4 hv = lds128(slot + 32 * STEP + lane * 16);
        sts128(base + p.side_off + ss * p.side_stage_bytes + (uint32_t)r * 16, hv);
        __syncwarp();
        if (lane == 0) mbar_arrive(side_full + 8 * ss);
      }
      XNQ_TACC(0);
      if (i >= BS) alive = mbar_wait_warp(mma_done + 8 * (2 * bs), a_ph ^ 1u, 2u) && mbar_wait_warp(mma_done + 8 * (2 * bs + 1), a_ph ^ 1u, 2u); // both halves of the stage have been multiplied
      XNQ_TACC(3);
      if (!alive) break;
#pragma unroll
      for (int h = 0; h < 2; h++) {
        uint4 lo[4], hi[4];
        Conv::run(slot + (uint32_t)lane * STEP, lane, h, 0, lo);
        Conv::run(slot + (uint32_t)lane * STEP, lane, h, 1, hi);
        const uint32_t dst_row = base + p.a_off + (2 * bs + h) * A_STAGE_BYTES + (uint32_t)r * 128;
#pragma unroll
        for (int c = 0; c < 4; c++) {
          sts128(dst_row + (uint32_t)((c ^ sw) << 4), lo[c]);
          sts128(dst_row + (uint32_t)(((4 + c) ^ sw) << 4), hi[c]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> visible to the tensor core
      __syncwarp(); // every lane has stored its row and has read all it needs of the slot
      if (lane == 0) mbar_arrive(a_full + 8 * bs);
      if (l_i < nunits) issue(); // into the slot just read
      cp_async_commit();
      if (threadIdx.x == CONV_WARP0 * 32) XNQ_TL(3, i);
      if (++rs == D) rs = 0;
      for (int t = 0; t < 2; t++)
        if (++bs == BS) bs = 0, a_ph ^= 1u;
    }
    cp_async_wait(0); // nothing may be in flight into this CTA's shared memory when it exits
    XNQ_TDUMP(12, threadIdx.x == CONV_WARP0 * 32);
  } else if (warp - DRAIN_WARP0 < 2 * DWG) {
    // ---- drain: group h (DWG warps) owns half step h of every 256-k step and the accumulator buffers of its parity. Warp
    // quarter q reads accumulator lanes 32q.. (weight rows); with eight warps per group the two warps of a quarter split the
    // columns. Each group keeps its own f32 sums; at the end of a segment group 1 hands its sums to group 0 through scratch
    // memory. ----
    const int dwi = warp - DRAIN_WARP0;
    const int q = warp & 3, h = dwi / DWG, cg = (dwi % DWG) >> 2;
    const int c0 = cg * NPT;
    const int et = threadIdx.x - DRAIN_WARP0 * 32; // 0..511
    pdl_wait(); // the kernel that prepares the activations also zeroes the tiles' tickets
#ifdef XNQ_DEV_TRACE
    if (blockIdx.x == 0 && threadIdx.x == DRAIN_WARP0 * 32) { unsigned long long g_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_)); g_imma_trace[28] = (long long)g_; }
#endif
    bool alive = true;
    int tile = tile0, kt = kt0;
    float acc[NPT];
#pragma unroll
    for (int c = 0; c < NPT; c++) acc[c] = 0.f;
    int seg_kt0 = kt0; // first step of the current segment inside its tile
    float *pair = p.pair_scratch + (size_t)blockIdx.x * NP * TILE_N; // group 1 -> group 0
    XNQ_TDECL;
    int bs = 0, nb = 0;  // i % BS, i % (NB / 2)
    uint32_t a_ph = 0;   // (i / BS) & 1
    for (int i = 0; i < nunits; i++) {
      const int ss = i % SIDE_STAGES;
      const int sa = 2 * bs + h, buf = 2 * nb + h;
      XNQ_TACC(0);
      if (alive) alive = mbar_wait_warp(side_full + 8 * ss, (i / SIDE_STAGES) & 1, 8u);
      XNQ_TACC(1);
      const uint32_t side = base + p.side_off + ss * p.side_stage_bytes;
      uint4 hdr = make_uint4(0, 0, 0, 0);
      if (alive) hdr = lds128(side + (uint32_t)(32 * q + lane) * 16);
      if (alive) alive = mbar_wait_warp(mma_done + 8 * sa, a_ph, 8u);
      XNQ_TACC(2);
      if (threadIdx.x == DRAIN_WARP0 * 32) XNQ_TL(6, i);
      if (alive) {
        tc_fence_after();
        const uint32_t taddr = tmem_d + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * BUF_COLS + c0);
#pragma unroll
        for (int ch = 0; ch < NPT / CH; ch++) { // eight columns at a time keeps the slices' values within the register budget
          uint32_t v[4][CH];
#pragma unroll
          for (int s = 0; s < 4; s++) tmem_ld<CH>(taddr + (uint32_t)(s * NP + ch * CH), v[s]);
          tmem_ld_wait();
          XNQ_TACC(3);
          if (ch == NPT / CH - 1) { // every value of the buffer this warp needs is in registers: it may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + 8 * buf);
          }
          Drain<CH>::run(hdr, side + HDR_BYTES, h, c0 + ch * CH, v, acc + ch * CH);
        }
      }
      __syncwarp();
      if (alive && lane == 0) mbar_arrive(side_empty + 8 * ss);
      if (threadIdx.x == DRAIN_WARP0 * 32) XNQ_TL(7, i);
      // ---- end of a segment (the tile's last step, or this CTA's last unit): store or hand over the sums ----
      const bool tile_end = kt == KT - 1, range_end = i == nunits - 1;
      if (tile_end || range_end) {
        const int64_t row = (int64_t)tile * TILE_N + 32 * q + lane;
        // group 1's sums (the odd half steps) join group 0's (the even ones): always even + odd, whatever the timing
        if (h == 1) {
#pragma unroll
          for (int c = 0; c < NPT; c++) pair[(size_t)(c0 + c) * TILE_N + 32 * q + lane] = acc[c];
          __threadfence_block();
        }
        asm volatile("bar.sync 1, %0;" ::"n"(2 * DWG * 32) : "memory");
        if (h == 0) {
#pragma unroll
          for (int c = 0; c < NPT; c++) acc[c] += pair[(size_t)(c0 + c) * TILE_N + 32 * q + lane];
        }
        const bool whole = seg_kt0 == 0 && tile_end;
        if (whole) {
          if (h == 0 && alive && row < p.w.n) {
#pragma unroll
            for (int c = 0; c < NPT; c++) {
              const int64_t col = c0 + c;
              if (col < p.m) {
                const int64_t idx = col * p.ldy + row;
                if (p.y_dtype == XNQ_F32) static_cast<float *>(p.y)[idx] = acc[c];
                else if (p.y_dtype == XNQ_F16) static_cast<__half *>(p.y)[idx] = __float2half_rn(acc[c]);
                else static_cast<__nv_bfloat16 *>(p.y)[idx] = __float2bfloat16_rn(acc[c]);
              }
            }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(2 * DWG * 32) : "memory"); // group 0 has read the scratch: it may be rewritten
        } else {
          // this CTA's first segment (it starts where the CTA's range starts) uses scratch slot 2c, a later one 2c + 1
          const int seg_u0 = tile * KT + seg_kt0;
          float *mine = p.partials + ((size_t)2 * blockIdx.x + (seg_u0 == u0 ? 0 : 1)) * NP * TILE_N;
          if (h == 0) {
#pragma unroll
            for (int c = 0; c < NPT; c++) mine[(size_t)(c0 + c) * TILE_N + 32 * q + lane] = acc[c];
            __threadfence();
          }
          asm volatile("bar.sync 1, %0;" ::"n"(2 * DWG * 32) : "memory");
          if (et == 0) s_ticket = atomicAdd(p.tile_cnt + tile, 1u);
          asm volatile("bar.sync 1, %0;" ::"n"(2 * DWG * 32) : "memory");
          const unsigned int ticket = s_ticket;
          asm volatile("bar.sync 1, %0;" ::"n"(2 * DWG * 32) : "memory"); // s_ticket may be rewritten from here on
          const int t_u0 = tile * KT, t_u1 = t_u0 + KT;
          const int c_first = cta_of(t_u0, p.units_q, p.units_r), c_last = cta_of(t_u1 - 1, p.units_q, p.units_r);
          if (et == 0 && (int)ticket == c_last - c_first) p.tile_cnt[tile] = 0u; // every part has its ticket: the word is zero again for the next call
          if (h == 0 && (int)ticket == c_last - c_first) { // the last part to arrive adds all parts in k order
            __threadfence();
            float (&sum)[NPT] = acc; // the segment's own sums are in its scratch slot by now
#pragma unroll
            for (int c = 0; c < NPT; c++) sum[c] = 0.f;
            for (int cc = c_first; cc <= c_last; cc++) {
              const int cu0 = cta_first_unit(cc, p.units_q, p.units_r);
              const float *part = p.partials + ((size_t)2 * cc + (cu0 >= t_u0 ? 0 : 1)) * NP * TILE_N;
#pragma unroll
              for (int c = 0; c < NPT; c++) sum[c] += __ldcg(part + (size_t)(c0 + c) * TILE_N + 32 * q + lane);
            }
            if (row < p.w.n) {
#pragma unroll
              for (int c = 0; c < NPT; c++) {
                const int64_t col = c0 + c;
                if (col < p.m) {
                  const int64_t idx = col * p.ldy + row;
                  if (p.y_dtype == XNQ_F32) static_cast<float *>(p.y)[idx] = sum[c];
                  else if (p.y_dtype == XNQ_F16) static_cast<__half *>(p.y)[idx] = __float2half_rn(sum[c]);
                  else static_cast<__nv_bfloat16 *>(p.y)[idx] = __float2bfloat16_rn(sum[c]);
                }
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < NPT; c++) acc[c] = 0.f;
        seg_kt0 = 0;
      }
      if (++kt == KT) {
        kt = 0;
        tile++;
      }
      if (++bs == BS) bs = 0, a_ph ^= 1u;
      if (2 * ++nb == NB) nb = 0;
    }
    XNQ_TDUMP(18, threadIdx.x == DRAIN_WARP0 * 32);
  }

  tc_fence_before();
  __syncthreads();
#ifdef XNQ_DEV_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) g_imma_trace[30] = nunits;
  XNQ_GT(27);
#endif
  if (warp == MMA_WARP) tmem_dealloc(tmem_d, TMEM_COLS);
}

// =====================================================================================================================
// Q4_K with the sub-block scales folded into the weight operand.
//
// The kernel above drains one accumulator slice per 32-element block, because a block's scale cannot be applied on the
// tensor core. For Q4_K the scales are small integers: a code q (0..15) times its 6-bit sub-block scale sc (0..63) is an
// integer below 1024, and written as q = 4 q_hi + q_lo (two bits each) both q_lo sc and q_hi sc fit one unsigned byte
// (<= 189). So the converters write TWO operand planes, P_lo = q_lo sc and P_hi = q_hi sc (one packed multiply per four
// codes, no carries between bytes), the MMAs ACCUMULATE over the four sub-blocks of a half step,
//     D_lo = sum_i P_lo[r, i] a[c, i],  D_hi likewise,    sum_g sc_g sum_{i in g} q_i a_i = 4 D_hi + D_lo   (exact integers),
// and the drain applies d, d_min and the activation scale once per 256-element block, as the CPU code does
// (k_quants.rs:1380-1410). Per 256-k step that is 16 MMAs instead of 8, issued by four threads (plane x half step; an
// MMA of this shape costs its issuing thread 134 cycles but several threads issue concurrently), and 4 accumulator
// slices to drain instead of 8, with the integer scale multiplies gone from the drain, which is what bounded the kernel
// above (instruction issue). 21 warps: activation producer, 4 MMA issuers, 8 converter warps (group h converts half h of
// every step into a ring of four half-step stages), 8 drain warps (two groups that take alternate steps; a thread owns
// one weight row and all NP activation columns). NP is 16 or 32; larger batches run in passes of 32 rows.
// =====================================================================================================================
constexpr int F_ISSUERS = 4, F_CONV_WARPS = 8, F_DRAIN_WARPS = 8;
constexpr int F_ACT_WARP = 0, F_MMA_WARP0 = 1, F_CONV_WARP0 = F_MMA_WARP0 + F_ISSUERS, F_DRAIN_WARP0 = F_CONV_WARP0 + F_CONV_WARPS;
constexpr int F_NTHREADS = (F_DRAIN_WARP0 + F_DRAIN_WARPS) * 32; // 672
constexpr int F_RING = 3;                         // stages of the rings that are freed by the drain (activation operand, scale bytes and records)
constexpr int F_ASTAGES = 4;                      // half-step stages of the weight operand (two steps), two planes each
constexpr int F_A_STAGE_BYTES = 2 * A_STAGE_BYTES; // plane lo, plane hi
constexpr uint32_t F_SLOT = 32 * 64 + 512;        // a converter warp's raw slot: 64 code bytes of the half step per row, then the rows' 16 header bytes

// kind::i8 with an UNSIGNED A operand (the scaled codes reach 189) and a signed B operand
__device__ __forceinline__ uint32_t idesc_u8s8(int umma_n) {
  return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);
}
__device__ __forceinline__ void umma_i8_acc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// a ring position: index in 0..n-1 and the parity of the lap, advanced without a division
struct RingPos {
  int idx;
  uint32_t ph;
  __device__ __forceinline__ void advance(int by, int n) {
    idx += by;
    if (idx >= n) idx -= n, ph ^= 1u;
  }
};

template <int NP>
__global__ void __launch_bounds__(F_NTHREADS, 1) imma_q4k_fold_kernel(const __grid_constant__ ImmaArgs p) {
  constexpr int NBUF = TMEM_COLS / (4 * NP) > 8 ? 8 : TMEM_COLS / (4 * NP); // accumulator buffers of one step (four slices): 8 or 4, a power of two
  constexpr int BUF_COLS = 4 * NP;
  constexpr int CH = 8; // columns read back at a time
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // barriers: b_full, side_full, side_empty [F_RING]; a_full [F_ASTAGES]; acc_full, acc_empty [8] (NBUF of them in use)
  __shared__ __align__(8) uint64_t bars[3 * F_RING + F_ASTAGES + 16];
  __shared__ uint32_t tmem_slot;
  __shared__ unsigned int s_ticket;
  const uint32_t b_full = smem_u32(bars), side_full = b_full + 8 * F_RING, side_empty = side_full + 8 * F_RING, a_full = side_empty + 8 * F_RING,
                 acc_full = a_full + 8 * F_ASTAGES, acc_empty = acc_full + 64;
  // One commit per issuer and step, on the step's accumulator buffer (acc_full, all four issuers): it tells the drain that the
  // slices are written and the converters that the operand stages of that step have been read. A barrier per operand stage
  // would be lapped: the issuers may run NBUF steps ahead of the drain, and a waiter that misses two phases waits for ever.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = p.raw_stages; // raw slots per converter warp
  const int KT = p.nsteps;
  const int u0 = cta_first_unit((int)blockIdx.x, p.units_q, p.units_r);
  const int nunits = p.units_q + ((int)blockIdx.x < p.units_r ? 1 : 0);
  const int tile0 = u0 / KT, kt0 = u0 - tile0 * KT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F_RING; s++) {
      mbar_init(b_full + 8 * s, 1);
      mbar_init(side_full + 8 * s, 1 + F_CONV_WARPS / 2); // the producer's transaction + the four converter warps of half 0, which copy the header bytes
      mbar_init(side_empty + 8 * s, F_DRAIN_WARPS / 2);   // the step's drain group
    }
    for (int s = 0; s < F_ASTAGES; s++) mbar_init(a_full + 8 * s, F_CONV_WARPS / 2); // the four converter warps of the half step
    for (int s = 0; s < 8; s++) {
      mbar_init(acc_full + 8 * s, F_ISSUERS);
      mbar_init(acc_empty + 8 * s, F_DRAIN_WARPS / 2);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == F_MMA_WARP0) {
    tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents();
  const uint32_t tmem_d = tmem_slot;

  if (warp == F_ACT_WARP) {
    // ---- activation producer ----
    if (lane == 0) {
      for (int st = 0; st < p.nstreams; st++) { // the CTA's share of the weight's bytes into L2, in long contiguous runs
        const unsigned long long o0 = p.pf_share[st] * blockIdx.x, o1 = min(o0 + p.pf_share[st], p.pf_bytes[st]);
        for (unsigned long long o = o0; o < o1; o += PF_CHUNK) bulk_prefetch_l2(p.pf_base[st] + o, (uint32_t)min((unsigned long long)PF_CHUNK, o1 - o));
      }
      pdl_wait();
      int kt = kt0;
      RingPos rp{0, 0};
      for (int i = 0; i < nunits; i++) {
        // the stage was last used by step i - 3; it is free once that step's drain group has read its records, which also
        // means the step's MMAs have read the activation operand
        if (i >= F_RING && !mbar_wait(side_empty + 8 * rp.idx, rp.ph ^ 1u, 1u)) break;
        mbar_expect_tx(b_full + 8 * rp.idx, p.b_stage_bytes);
        mbar_expect_tx(side_full + 8 * rp.idx, (uint32_t)NP * 32u);
        bulk_g2s(base + p.b_off + rp.idx * p.b_stage_bytes, p.bimg + ((size_t)kt * 2) * (NP * 128), p.b_stage_bytes, b_full + 8 * rp.idx);
        bulk_g2s(base + p.side_off + rp.idx * p.side_stage_bytes + HDR_BYTES, p.meta + (size_t)kt * (NP * 32), (uint32_t)NP * 32u, side_full + 8 * rp.idx);
        if (++kt == KT) kt = 0;
        rp.advance(1, F_RING);
      }
    }
  } else if (warp < F_CONV_WARP0) {
    // ---- MMA issuers: plane pl (0: q_lo sc, 1: q_hi sc) of half step h ----
    const int pl = (warp - F_MMA_WARP0) >> 1, h = (warp - F_MMA_WARP0) & 1;
    if (lane == 0) {
      const uint32_t idesc = idesc_u8s8(NP);
      RingPos rp{0, 0}; // step i in the drain-freed ring
      uint32_t acc_ph = 0;
      for (int i = 0; i < nunits; i++) {
        const int buf = i & (NBUF - 1), st = 2 * (i & 1) + h; // half step j = 2 i + h uses operand stage j % 4
        if (!mbar_wait(b_full + 8 * rp.idx, rp.ph, 4u)) break;
        if (!mbar_wait(a_full + 8 * st, (uint32_t)(i >> 1) & 1u, 4u)) break;
        if (i >= NBUF && !mbar_wait(acc_empty + 8 * buf, acc_ph ^ 1u, 4u)) break; // the drain of the buffer's previous step
        tc_fence_after();
        const uint64_t adesc = smem_desc_sw128(base + p.a_off + st * F_A_STAGE_BYTES + pl * A_STAGE_BYTES);
        const uint64_t bdesc = smem_desc_sw128(base + p.b_off + rp.idx * p.b_stage_bytes + h * (NP * 128));
        const uint32_t dcol = tmem_d + (uint32_t)(buf * BUF_COLS + (pl * 2 + h) * NP);
#pragma unroll
        for (int q = 0; q < 4; q++) umma_i8_acc(dcol, adesc + (uint64_t)(q * 2), bdesc + (uint64_t)(q * 2), idesc, q > 0 ? 1u : 0u);
        umma_commit(acc_full + 8 * buf);
        rp.advance(1, F_RING);
        if (buf == NBUF - 1) acc_ph ^= 1u;
      }
    }
  } else if (warp < F_DRAIN_WARP0) {
    // ---- converters: group h (four warps, one thread per weight row) writes both planes of half step h of every step ----
    const int cw = warp - F_CONV_WARP0;
    const int r0 = (cw & 3) * 32, r = r0 + lane, h = cw >> 2;
    const int sw = r & 7;
    const uint32_t slot0 = base + p.raw_off0 + (uint32_t)(cw * D) * F_SLOT;
    const int64_t n = p.w.n;
    int l_i = 0, l_tile = tile0, l_kt = kt0, l_s = 0;
    auto issue = [&]() { // lane l copies chunk l % 4 of row q * 8 + l / 4 in instruction q; then its own row's header
      const uint32_t dst = slot0 + (uint32_t)l_s * F_SLOT;
      const int c = lane & 3;
      const uint32_t in_row = (uint32_t)l_kt * 144u + 16u + (uint32_t)(h * 64 + c * 16);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int rw = q * 8 + (lane >> 2);
        const int64_t grow = (int64_t)l_tile * TILE_N + r0 + rw;
        const bool ok = grow < n;
        cp_async16(dst + (uint32_t)(rw * 64 + ((c ^ (rw & 3)) << 4)), p.src[0] + (size_t)(ok ? grow : n - 1) * p.row_bytes[0] + in_row, ok ? 16u : 0u);
      }
      const int64_t grow = (int64_t)l_tile * TILE_N + r;
      cp_async16(dst + 2048 + lane * 16, p.src[0] + (size_t)(grow < n ? grow : n - 1) * p.row_bytes[0] + (size_t)l_kt * 144u, grow < n ? 16u : 0u);
      l_i++;
      if (++l_kt == KT) l_kt = 0, l_tile++;
      if (++l_s == D) l_s = 0;
    };
    for (int u = 0; u < D; u++) {
      if (l_i < nunits) issue();
      cp_async_commit();
    }
    bool alive = true;
    int rs = 0;
    RingPos rp{0, 0};
    for (int i = 0; i < nunits && alive; i++) {
      const int st = 2 * (i & 1) + h;
      cp_async_wait(D - 1);
      __syncwarp();
      const uint32_t slot = slot0 + (uint32_t)rs * F_SLOT;
      const uint4 hdr = lds128(slot + 2048 + lane * 16);
      if (h == 0) { // hand the row's header on to the drain
        if (i >= F_RING) alive = mbar_wait_warp(side_empty + 8 * rp.idx, rp.ph ^ 1u, 2u);
        if (!alive) break;
        sts128(base + p.side_off + rp.idx * p.side_stage_bytes + (uint32_t)r * 16, hdr);
        __syncwarp();
        if (lane == 0) mbar_arrive(side_full + 8 * rp.idx);
      }
      // the stage's previous half step belongs to step i - 2: all of that step's MMAs have been committed
      if (i >= 2) alive = mbar_wait_warp(acc_full + 8 * ((i - 2) & (NBUF - 1)), (uint32_t)((i - 2) / NBUF) & 1u, 2u);
      if (!alive) break;
      // the four sub-block scales of this half step: fields 2h and 2h + 1 of the repacked header
      const uint32_t lo32 = h ? __funnelshift_r(hdr.z, hdr.w, 16) : hdr.y;
      const uint32_t hi16 = h ? (hdr.w >> 16) : (hdr.z & 0xffffu);
      const uint32_t f0 = lo32 & 0xffffffu, f1 = __funnelshift_r(lo32, hi16, 24) & 0xffffffu;
      const uint32_t sc[4] = {f0 & 63u, (f0 >> 6) & 63u, f1 & 63u, (f1 >> 6) & 63u};
      const uint32_t row = slot + (uint32_t)lane * 64;
      const uint4 raw[4] = {raw_chunk<64>(row, lane, 0), raw_chunk<64>(row, lane, 1), raw_chunk<64>(row, lane, 2), raw_chunk<64>(row, lane, 3)};
      const uint32_t a_stage = base + p.a_off + st * F_A_STAGE_BYTES + (uint32_t)r * 128;
#pragma unroll
      for (int pl = 0; pl < 2; pl++) {
#pragma unroll
        for (int pair = 0; pair < 2; pair++) { // 32-byte chunk `pair` of the half step: sub-blocks 2 pair (low nibbles) and 2 pair + 1 (high nibbles)
#pragma unroll
          for (int nib = 0; nib < 2; nib++) {
            const int sh = 4 * nib + 2 * pl;
            const uint32_t m = sc[2 * pair + nib];
#pragma unroll
            for (int half16 = 0; half16 < 2; half16++) { // the chunk's first and second 16 bytes: elements 0..15 and 16..31 of the sub-block
              const uint4 w = raw[2 * pair + half16];
              const uint4 o = make_uint4(((w.x >> sh) & 0x03030303u) * m, ((w.y >> sh) & 0x03030303u) * m, ((w.z >> sh) & 0x03030303u) * m,
                                         ((w.w >> sh) & 0x03030303u) * m);
              const int chunk = (2 * pair + nib) * 2 + half16; // 16-byte chunk of the 128-byte operand row
              sts128(a_stage + pl * A_STAGE_BYTES + (uint32_t)((chunk ^ sw) << 4), o);
            }
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(a_full + 8 * st);
      if (l_i < nunits) issue();
      cp_async_commit();
      if (++rs == D) rs = 0;
      rp.advance(1, F_RING);
    }
    cp_async_wait(0);
  } else {
    // ---- drain: group dg (four warps, a thread per weight row, all NP columns) takes the steps i = dg, dg + 2, ... ----
    const int dwi = warp - F_DRAIN_WARP0;
    const int q = warp & 3, dg = dwi >> 2;
    const int et = threadIdx.x - F_DRAIN_WARP0 * 32; // 0..255
    pdl_wait(); // the kernel that prepares the activations also zeroes the tiles' tickets
    bool alive = true;
    int tile = tile0, kt = kt0;
    float acc[NP];
#pragma unroll
    for (int c = 0; c < NP; c++) acc[c] = 0.f;
    int seg_kt0 = kt0;
    float *pair = p.pair_scratch + (size_t)blockIdx.x * NP * TILE_N;
    RingPos rp{0, 0};
    for (int i = 0; i < nunits; i++) {
      const int buf = i & (NBUF - 1);
      if ((i & 1) == dg) {
        if (alive) alive = mbar_wait_warp(side_full + 8 * rp.idx, rp.ph, 8u);
        const uint32_t side = base + p.side_off + rp.idx * p.side_stage_bytes;
        uint4 hdr = make_uint4(0, 0, 0, 0);
        if (alive) hdr = lds128(side + (uint32_t)(32 * q + lane) * 16);
        if (alive) alive = mbar_wait_warp(acc_full + 8 * buf, (uint32_t)(i / NBUF) & 1u, 8u);
        if (alive) {
          tc_fence_after();
          const __half2 dm = *reinterpret_cast<const __half2 *>(&hdr.x);
          const float d = __low2float(dm), dmin = __high2float(dm);
          // the eight 6-bit mins as bytes: fields F0..F3 hold mn[2g] at bit 12 and mn[2g+1] at bit 18
          const uint32_t F0 = hdr.y & 0xffffffu, F1 = __funnelshift_r(hdr.y, hdr.z, 24) & 0xffffffu, F2 = __funnelshift_r(hdr.z, hdr.w, 16) & 0xffffffu, F3 = hdr.w >> 8;
          const uint32_t mins0 = ((F0 >> 12) & 63u) | (((F0 >> 18) & 63u) << 8) | (((F1 >> 12) & 63u) << 16) | (((F1 >> 18) & 63u) << 24);
          const uint32_t mins1 = ((F2 >> 12) & 63u) | (((F2 >> 18) & 63u) << 8) | (((F3 >> 12) & 63u) << 16) | (((F3 >> 18) & 63u) << 24);
          const uint32_t taddr = tmem_d + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * BUF_COLS);
#pragma unroll
          for (int ch = 0; ch < NP / CH; ch++) {
            uint32_t v[4][CH]; // slices: plane lo half 0, lo half 1, hi half 0, hi half 1
#pragma unroll
            for (int sl = 0; sl < 4; sl++) tmem_ld<CH>(taddr + (uint32_t)(sl * NP + ch * CH), v[sl]);
            tmem_ld_wait();
            if (ch == NP / CH - 1) { // every value of the buffer is in registers: it may be overwritten
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(acc_empty + 8 * buf);
            }
#pragma unroll
            for (int c = 0; c < CH; c++) {
              const uint32_t rec = side + HDR_BYTES + (uint32_t)(ch * CH + c) * 32;
              const uint4 bs = lds128(rec); // {lo bytes half 0, hi bytes half 0, lo bytes half 1, hi bytes half 1} of the activations' 32-sums
              const float da = __uint_as_float(lds32(rec + 16));
              const int isum = 4 * ((int)v[2][c] + (int)v[3][c]) + ((int)v[0][c] + (int)v[1][c]);
              const int msum = dp4a_uu(mins0, bs.x, dp4a_uu(mins1, bs.z, 0)) + 128 * dp4a_us(mins0, bs.y, dp4a_us(mins1, bs.w, 0));
              acc[ch * CH + c] += da * (d * (float)isum - dmin * (float)msum);
            }
          }
        }
        __syncwarp();
        if (alive && lane == 0) mbar_arrive(side_empty + 8 * rp.idx);
      }
      // ---- end of a segment (the tile's last step, or this CTA's last unit): store or hand over the sums ----
      const bool tile_end = kt == KT - 1, range_end = i == nunits - 1;
      if (tile_end || range_end) {
        const int64_t row = (int64_t)tile * TILE_N + 32 * q + lane;
        if (dg == 1) { // the odd steps' sums join the even ones': always even + odd, whatever the timing
#pragma unroll
          for (int c = 0; c < NP; c++) pair[(size_t)c * TILE_N + 32 * q + lane] = acc[c];
          __threadfence_block();
        }
        asm volatile("bar.sync 1, %0;" ::"n"(F_DRAIN_WARPS * 32) : "memory");
        if (dg == 0) {
#pragma unroll
          for (int c = 0; c < NP; c++) acc[c] += pair[(size_t)c * TILE_N + 32 * q + lane];
        }
        const bool whole = seg_kt0 == 0 && tile_end;
        if (whole) {
          if (dg == 0 && alive && row < p.w.n) {
#pragma unroll
            for (int c = 0; c < NP; c++) {
              if (c < p.m) {
                const int64_t idx = (int64_t)c * p.ldy + row;
                if (p.y_dtype == XNQ_F32) static_cast<float *>(p.y)[idx] = acc[c];
                else if (p.y_dtype == XNQ_F16) static_cast<__half *>(p.y)[idx] = __float2half_rn(acc[c]);
                else static_cast<__nv_bfloat16 *>(p.y)[idx] = __float2bfloat16_rn(acc[c]);
              }
            }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(F_DRAIN_WARPS * 32) : "memory"); // group 0 has read the scratch: it may be rewritten
        } else {
          const int seg_u0 = tile * KT + seg_kt0;
          float *mine = p.partials + ((size_t)2 * blockIdx.x + (seg_u0 == u0 ? 0 : 1)) * NP * TILE_N;
          if (dg == 0) {
#pragma unroll
            for (int c = 0; c < NP; c++) mine[(size_t)c * TILE_N + 32 * q + lane] = acc[c];
            __threadfence();
          }
          asm volatile("bar.sync 1, %0;" ::"n"(F_DRAIN_WARPS * 32) : "memory");
          if (et == 0) s_ticket = atomicAdd(p.tile_cnt + tile, 1u);
          asm volatile("bar.sync 1, %0;" ::"n"(F_DRAIN_WARPS * 32) : "memory");
          const unsigned int ticket = s_ticket;
          asm volatile("bar.sync 1, %0;" ::"n"(F_DRAIN_WARPS * 32) : "memory");
          const int t_u0 = tile * KT, t_u1 = t_u0 + KT;
          const int c_first = cta_of(t_u0, p.units_q, p.units_r), c_last = cta_of(t_u1 - 1, p.units_q, p.units_r);
          if (et == 0 && (int)ticket == c_last - c_first) p.tile_cnt[tile] = 0u; // every part has its ticket: the word is zero again for the next call
          if (dg == 0 && (int)ticket == c_last - c_first) { // the last part to arrive adds all parts in k order
            __threadfence();
#pragma unroll
            for (int c = 0; c < NP; c++) acc[c] = 0.f;
            for (int cc = c_first; cc <= c_last; cc++) {
              const int cu0 = cta_first_unit(cc, p.units_q, p.units_r);
              const float *part = p.partials + ((size_t)2 * cc + (cu0 >= t_u0 ? 0 : 1)) * NP * TILE_N;
#pragma unroll
              for (int c = 0; c < NP; c++) acc[c] += __ldcg(part + (size_t)c * TILE_N + 32 * q + lane);
            }
            if (row < p.w.n) {
#pragma unroll
              for (int c = 0; c < NP; c++) {
                if (c < p.m) {
                  const int64_t idx = (int64_t)c * p.ldy + row;
                  if (p.y_dtype == XNQ_F32) static_cast<float *>(p.y)[idx] = acc[c];
                  else if (p.y_dtype == XNQ_F16) static_cast<__half *>(p.y)[idx] = __float2half_rn(acc[c]);
                  else static_cast<__nv_bfloat16 *>(p.y)[idx] = __float2bfloat16_rn(acc[c]);
                }
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < NP; c++) acc[c] = 0.f;
        seg_kt0 = 0;
      }
      if (++kt == KT) kt = 0, tile++;
      rp.advance(1, F_RING);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == F_MMA_WARP0) tmem_dealloc(tmem_d, TMEM_COLS);
}

// ---- activations: quantize (or take an activation image), lay out as the MMA's B operand, write the records ----
// CTAs of 256 threads over (activation row of the padded pass, 2048-element stretch of k); rows >= m are zero.
// Thread t handles elements 8t..8t+7 of a stretch; a warp covers one 256-element block.
template <int ACT, typename XT>
__global__ void __launch_bounds__(256) imma_prepare(const XT *__restrict__ x, const int8_t *__restrict__ img_q, const float *__restrict__ img_d,
                                                    const int16_t *__restrict__ img_b, int64_t m, int64_t k, int64_t ldx, int NP, int nsteps,
                                                    uint8_t *__restrict__ bimg, uint8_t *__restrict__ meta, unsigned int *__restrict__ tile_cnt, int tiles) {
  pdl_launch_dependents(); // the matmul kernel may start its set-up and its weight loads now
  pdl_wait();              // x may be the previous kernel's output; the scratch may still be read by the previous call
  XNQ_GT(24);
  const int row = blockIdx.x;
  if (blockIdx.x == 0 && blockIdx.y == 0)
    for (int i = threadIdx.x; i < tiles; i += blockDim.x) tile_cnt[i] = 0;
  const int lane = threadIdx.x & 31;
  const int64_t kpad = (int64_t)nsteps * 256;
  const int nblk_act = (int)(k / (ACT == XNQ_Q8_0 ? QK : QK_K));
  for (int64_t base = (int64_t)blockIdx.y * 2048; base < kpad; base += (int64_t)gridDim.y * 2048) {
    const int64_t k8 = base + (int64_t)threadIdx.x * 8;
    if (base + (int64_t)(threadIdx.x & ~31) * 8 >= kpad) break; // whole warps leave together
    uint32_t lo = 0, hi = 0;
    float d = 0.f;
    int sum16 = 0;
    const bool valid = row < m && k8 < k;
    if (img_q) {
      if (valid) {
        const uint2 c = *reinterpret_cast<const uint2 *>(img_q + (int64_t)row * k + k8);
        lo = c.x, hi = c.y;
        d = img_d[(int64_t)row * nblk_act + (ACT == XNQ_Q8_0 ? k8 / QK : k8 / QK_K)];
        sum16 = img_b[(int64_t)row * (k / 16) + k8 / 16];
      }
    } else {
      float v[8];
      if (valid) load8(x + (int64_t)row * ldx + k8, v);
      else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = 0.f;
      }
      const Quant8 qv = ACT == XNQ_Q8_0 ? quantize8_q8_0(v, lane) : quantize8_q8k(v, lane);
      lo = qv.lo, hi = qv.hi, d = qv.d, sum16 = qv.sum16;
    }
    if (k8 < kpad) {
      // operand image: half step hs = k8 / 128, row `row`, 16-byte chunk (k8 % 128) / 16 swizzled with the row
      const int64_t hs = k8 >> 7;
      const int chunk = (int)((k8 & 127) >> 4);
      uint8_t *dst = bimg + (size_t)hs * (NP * 128) + (size_t)(row >> 3) * 1024 + (size_t)(row & 7) * 128 + (size_t)((chunk ^ (row & 7)) << 4) + (k8 & 8);
      *reinterpret_cast<uint2 *>(dst) = make_uint2(lo, hi);
      uint32_t *rec = reinterpret_cast<uint32_t *>(meta + ((size_t)(k8 >> 8) * NP + row) * 32);
      if (ACT == XNQ_Q8_0) {
        if ((lane & 3) == 0) rec[(k8 & 255) >> 5] = __float_as_uint(d); // eight f32 block scales (0 beyond k)
      } else {
        // 32-sums of the block's eight sub-blocks: lanes 4s .. 4s+3 hold sub-block s; sum16 is the pair sum on both lanes of a pair
        const int s32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 2);
        const int sub = lane >> 2;
        uint32_t lo_b = (lane & 3) == 0 ? ((uint32_t)(s32 & 127) << (8 * (sub & 3))) : 0u;
        uint32_t hi_b = (lane & 3) == 0 ? ((uint32_t)((s32 >> 7) & 0xff) << (8 * (sub & 3))) : 0u;
        // combine the four sub-blocks of each half of the block: lanes 0..15 -> words 0 / 1, lanes 16..31 -> words 2 / 3
#pragma unroll
        for (int off = 4; off <= 8; off <<= 1) {
          lo_b |= __shfl_xor_sync(0xffffffffu, lo_b, off);
          hi_b |= __shfl_xor_sync(0xffffffffu, hi_b, off);
        }
        if (lane == 0 || lane == 16) {
          rec[(lane >> 4) * 2] = lo_b;
          rec[(lane >> 4) * 2 + 1] = hi_b;
        }
        if (lane == 0) {
          rec[4] = __float_as_uint(d);
          rec[5] = rec[6] = rec[7] = 0u;
        }
      }
    }
  }
  XNQ_GT(25);
}

int g_sms = 0;
std::atomic<int> g_fold{1}; // Q4_K, imma_q4k_fold_kernel: 0 never, 1 for the batch sizes it is faster at, 2 whenever the weight is Q4_K

struct Plan {
  int NP, nsteps, tiles, grid;
  size_t bimg_bytes, meta_bytes, cnt_bytes, part_bytes, pair_bytes;
};
Plan plan_for(int64_t m, int64_t k, int64_t n) {
  Plan pl{};
  pl.NP = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
  pl.nsteps = (int)((k + 255) / 256);
  pl.tiles = (int)((n + TILE_N - 1) / TILE_N);
  const long long units = (long long)pl.tiles * pl.nsteps;
  pl.grid = (int)std::max<long long>(1, std::min<long long>(g_sms > 0 ? g_sms : 148, units / 2)); // at least two steps per CTA
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  pl.bimg_bytes = up((size_t)pl.nsteps * 2 * pl.NP * 128);
  pl.meta_bytes = up((size_t)pl.nsteps * pl.NP * 32);
  pl.cnt_bytes = up((size_t)pl.tiles * 4);
  pl.part_bytes = up((size_t)2 * (g_sms > 0 ? g_sms : 148) * pl.NP * TILE_N * 4);
  pl.pair_bytes = up((size_t)(g_sms > 0 ? g_sms : 148) * pl.NP * TILE_N * 4);
  return pl;
}

template <typename Conv, template <int> class Drain>
int launch_np(const ImmaArgs &a, int NP, unsigned grid, cudaStream_t s) {
  // programmatic stream serialization: the kernel starts while the one that prepares the activations still runs; only
  // its weight loads are issued before griddepcontrol.wait
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = IMMA_SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (NP == 16) XNQ_CUDA(cudaLaunchKernelEx(&cfg, imma_kernel<Conv, Drain, 16>, a));
  else if (NP == 32) XNQ_CUDA(cudaLaunchKernelEx(&cfg, imma_kernel<Conv, Drain, 32>, a));
  else XNQ_CUDA(cudaLaunchKernelEx(&cfg, imma_kernel<Conv, Drain, 64>, a));
  count_launch();
  return XNQ_OK;
}

template <typename Conv, template <int> class Drain>
int init_np() {
  XNQ_CUDA(cudaFuncSetAttribute(imma_kernel<Conv, Drain, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IMMA_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(imma_kernel<Conv, Drain, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IMMA_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(imma_kernel<Conv, Drain, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IMMA_SMEM));
  return XNQ_OK;
}

} // namespace

bool imma_supported(const WeightView &w, int64_t m) {
  if (g_sms <= 0 || m < 1 || w.n < 1) return false;
  if (w.dtype != XNQ_Q4_0 && w.dtype != XNQ_Q8_0 && w.dtype != XNQ_Q4K) return false;
  if (((w.n + TILE_N - 1) / TILE_N) * ((w.k + 255) / 256) >= (1ll << 30)) return false; // the (tile, step) space is indexed with 32-bit integers
  return true;
}

// scratch of one call: the activations' operand image and records, the split tiles' tickets and partial sums
size_t imma_workspace_bytes(int64_t m, int64_t k, int64_t n) {
  const Plan pl = plan_for(std::min<int64_t>(m, MAX_NP), k, n);
  return pl.bimg_bytes + pl.meta_bytes + pl.cnt_bytes + pl.part_bytes + pl.pair_bytes + 256;
}

// x: float activations [m, k] (x_dtype F32 / F16 / BF16, row stride ldx) or an activation image (XNQ_ACT_IMAGE) of m rows.
int launch_imma(const WeightView &w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy, void *workspace,
                cudaStream_t s) {
  const int64_t k = w.k;
  const int act = act_dtype_for(w.dtype);
  const size_t yes = type_size(y_dtype);
  // Q4_K: sub-block scales folded into the weight operand. Measured on the 14336 x 4096 weight: as fast as the per-block
  // kernel up to 16 rows, 8 % faster for 17..32, slower beyond (it runs in passes of 32 rows), so by default it takes 17..32.
  const int fold_opt = g_fold.load(std::memory_order_relaxed);
  const bool fold = w.dtype == XNQ_Q4K && (fold_opt == 2 || (fold_opt == 1 && m > 16 && m <= 32)) && !(x_dtype == XNQ_ACT_OPERAND && m > 32); // an operand image is one pass
  const int64_t pass_rows = fold ? 32 : MAX_NP;
  const bool operand = x_dtype == XNQ_ACT_OPERAND; // the activations arrive in the kernel's own layout, with their ticket words: no activation kernel
  if (operand && (act != XNQ_Q8K || k % 256 || m > pass_rows)) return fail(XNQ_ERR_UNSUPPORTED, "imma: an operand image serves Q8_K activations of one pass (m = %lld)", (long long)m);
  for (int64_t r0 = 0; r0 < m; r0 += pass_rows) { // passes of at most 64 (32) activation rows
    const int64_t rows = std::min<int64_t>(pass_rows, m - r0);
    const Plan pl = plan_for(rows, k, w.n);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    uint8_t *bimg = ws;
    uint8_t *meta = bimg + pl.bimg_bytes;
    unsigned int *cnt = reinterpret_cast<unsigned int *>(meta + pl.meta_bytes);
    float *partials = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(cnt) + pl.cnt_bytes); // always in the caller's workspace
    if (operand) {
      if (pl.tiles > OPERAND_MAX_TILES) return fail(XNQ_ERR_SIZE, "imma: an operand image has ticket words for %d tiles of 128 rows, the weight has %d", OPERAND_MAX_TILES, pl.tiles);
      uint8_t *img = static_cast<uint8_t *>(const_cast<void *>(x));
      cnt = reinterpret_cast<unsigned int *>(img);
      bimg = img + OPERAND_TICKET_BYTES;
      meta = bimg + operand_bimg_bytes(pl.NP, k);
    }
    // ---- activations ----
    const int8_t *iq = nullptr;
    const float *id = nullptr;
    const int16_t *ib = nullptr;
    if (x_dtype == XNQ_ACT_IMAGE) {
      const ActView av = act_view(const_cast<void *>(x), m, k, act);
      const int blk = act == XNQ_Q8_0 ? QK : QK_K;
      iq = av.q + r0 * k, id = av.d + r0 * (k / blk), ib = av.bsum + r0 * (k / 16);
    }
#define XNQ_IMMA_PREP(ACT, XT)                                                                                                          \
  XNQ_CUDA(launch_pdl(imma_prepare<ACT, XT>, dim3((unsigned)pl.NP, (unsigned)std::min<int64_t>(16, (k + 2047) / 2048)), dim3(256), 0, s,     \
                      iq ? nullptr : static_cast<const XT *>(x) + r0 * ldx, iq, id, ib, rows, k, ldx, pl.NP, pl.nsteps, bimg, meta, cnt, pl.tiles))
    if (operand) {
      // nothing to prepare
    } else if (act == XNQ_Q8_0) {
      if (x_dtype == XNQ_F16) XNQ_IMMA_PREP(XNQ_Q8_0, __half);
      else if (x_dtype == XNQ_BF16) XNQ_IMMA_PREP(XNQ_Q8_0, __nv_bfloat16);
      else XNQ_IMMA_PREP(XNQ_Q8_0, float);
    } else {
      if (x_dtype == XNQ_F16) XNQ_IMMA_PREP(XNQ_Q8K, __half);
      else if (x_dtype == XNQ_BF16) XNQ_IMMA_PREP(XNQ_Q8K, __nv_bfloat16);
      else XNQ_IMMA_PREP(XNQ_Q8K, float);
    }
#undef XNQ_IMMA_PREP
    if (!operand) count_launch();

    ImmaArgs a{};
    a.w = w;
    a.bimg = bimg;
    a.meta = meta;
    a.y = static_cast<char *>(y) + (size_t)r0 * ldy * yes;
    a.y_dtype = y_dtype;
    a.ldy = ldy;
    a.m = rows;
    a.nsteps = pl.nsteps;
    a.tiles = pl.tiles;
    a.units = pl.tiles * pl.nsteps;
    a.units_q = a.units / pl.grid, a.units_r = a.units % pl.grid;
    a.tile_cnt = cnt;
    a.partials = partials;
    a.pair_scratch = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(partials) + pl.part_bytes);
    int rc, step_code; // step_code: code bytes per row and step
    switch (w.dtype) {
      case XNQ_Q4K:
        a.nstreams = 1, a.src[0] = w.qs, a.row_bytes[0] = (uint32_t)(k / QK_K * 144), a.step_bytes[0] = 144, a.code_off = 16, step_code = ConvQ4K::STEP;
        break;
      case XNQ_Q8_0:
        a.nstreams = 2, a.src[0] = w.qs, a.row_bytes[0] = (uint32_t)k, a.step_bytes[0] = 256, a.code_off = 0, step_code = ConvQ8_0::STEP;
        a.src[1] = reinterpret_cast<const uint8_t *>(w.d), a.row_bytes[1] = (uint32_t)(w.dstride * 2), a.step_bytes[1] = 16;
        break;
      case XNQ_Q4_0:
        a.nstreams = 2, a.src[0] = w.qs, a.row_bytes[0] = (uint32_t)(k / 2), a.step_bytes[0] = 128, a.code_off = 0, step_code = ConvQ4_0::STEP;
        a.src[1] = reinterpret_cast<const uint8_t *>(w.d), a.row_bytes[1] = (uint32_t)(w.dstride * 2), a.step_bytes[1] = 16;
        break;
      default: return fail(XNQ_ERR_DTYPE, "imma: dtype %d", w.dtype);
    }
    {
      size_t total = 0;
      for (int st = 0; st < a.nstreams; st++) total += (size_t)a.row_bytes[st] * (size_t)w.n;
      for (int st = 0; st < 2; st++) {
        a.pf_base[st] = st < a.nstreams ? a.src[st] : nullptr;
        a.pf_bytes[st] = st < a.nstreams && total <= PF_MAX_BYTES ? (unsigned long long)(((size_t)a.row_bytes[st] * (size_t)w.n) & ~(size_t)15) : 0ull;
#ifdef XNQ_DEV_TRACE
        if (const char *e = getenv("XNQ_IMMA_PF")) if (atoi(e) == 0) a.pf_bytes[st] = 0;
#endif
        a.pf_share[st] = ((a.pf_bytes[st] / (unsigned)pl.grid) + PF_CHUNK - 1) & ~(unsigned long long)(PF_CHUNK - 1);
      }
    }
    if (fold) {
      a.b_stage_bytes = (uint32_t)pl.NP * 256;
      a.side_stage_bytes = HDR_BYTES + (uint32_t)pl.NP * 32;
      a.a_off = 0;
      a.b_off = (uint32_t)F_ASTAGES * F_A_STAGE_BYTES;
      a.side_off = a.b_off + F_RING * a.b_stage_bytes;
      a.raw_off0 = (a.side_off + F_RING * a.side_stage_bytes + 127) & ~127u;
      const size_t left = IMMA_SMEM - 1024 - a.raw_off0;
      a.raw_stages = (int)std::min<size_t>(6, left / ((size_t)F_CONV_WARPS * F_SLOT)); // raw slots per converter warp
      if (a.raw_stages < 2) return fail(XNQ_ERR_SIZE, "imma: shared-memory plan does not fit");
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3((unsigned)pl.grid);
      cfg.blockDim = dim3(F_NTHREADS);
      cfg.dynamicSmemBytes = IMMA_SMEM;
      cfg.stream = s;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      profile_mark(s, true);
      if (pl.NP == 16) XNQ_CUDA(cudaLaunchKernelEx(&cfg, imma_q4k_fold_kernel<16>, a));
      else XNQ_CUDA(cudaLaunchKernelEx(&cfg, imma_q4k_fold_kernel<32>, a));
      count_launch();
      profile_mark(s, false);
      continue;
    }
    a.raw_stage_bytes = (uint32_t)(CONV_WARPS / 2) * (32u * (uint32_t)step_code + 512u); // a step in flight: four warp slots of the rows' code bytes and 16 scale bytes per row
    a.b_stage_bytes = (uint32_t)pl.NP * 256;
    a.side_stage_bytes = HDR_BYTES + (uint32_t)pl.NP * 32;
    // shared-memory plan: A stages (half steps) | B stages (half as many whole steps) | side stages | raw stages. The MMA
    // issuer bounds a step, so the converters and the drain need little slack (six half steps of operand image); what remains
    // goes to raw stages, which hide the memory latency.
    const size_t budget = IMMA_SMEM - 1024; // 1024: alignment slack of the base
    a.a_stages = 0;
    int as_order[3] = {6, 4, 8};
#ifdef XNQ_DEV_TRACE
    if (const char *e = getenv("XNQ_IMMA_AS")) as_order[0] = atoi(e);
#endif
    for (int ai = 0; ai < 3 && !a.a_stages; ai++) {
      const int as = as_order[ai];
      for (int rs = MAX_RAW_STAGES; rs >= 2 && !a.a_stages; rs -= 2) // even: the two converter groups own half of the slots each
        if ((size_t)as * A_STAGE_BYTES + (size_t)(as / 2) * a.b_stage_bytes + (size_t)SIDE_STAGES * a.side_stage_bytes + (size_t)rs * a.raw_stage_bytes + 256 <= budget &&
            (rs >= 4 || as == 4))
          a.a_stages = as, a.raw_stages = rs;
    }
    if (!a.a_stages) return fail(XNQ_ERR_SIZE, "imma: shared-memory plan does not fit");
    a.b_stages = a.a_stages / 2;
    a.a_off = 0;
    a.b_off = (uint32_t)a.a_stages * A_STAGE_BYTES;
    a.side_off = a.b_off + a.b_stages * a.b_stage_bytes;
    a.raw_off0 = (a.side_off + SIDE_STAGES * a.side_stage_bytes + 127) & ~127u;
    profile_mark(s, true);
    if (w.dtype == XNQ_Q4K) rc = launch_np<ConvQ4K, DrainQ4K>(a, pl.NP, (unsigned)pl.grid, s);
    else if (w.dtype == XNQ_Q8_0) rc = launch_np<ConvQ8_0, DrainBlockScaled>(a, pl.NP, (unsigned)pl.grid, s);
    else rc = launch_np<ConvQ4_0, DrainBlockScaled>(a, pl.NP, (unsigned)pl.grid, s);
    profile_mark(s, false);
    if (rc != XNQ_OK) return rc;
  }
  return XNQ_OK;
}

int imma_init(int device) {
  cudaDeviceProp prop;
  XNQ_CUDA(cudaGetDeviceProperties(&prop, device));
  g_sms = prop.multiProcessorCount;
  int rc;
  if ((rc = init_np<ConvQ4K, DrainQ4K>()) != XNQ_OK) return rc;
  XNQ_CUDA(cudaFuncSetAttribute(imma_q4k_fold_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IMMA_SMEM));
  XNQ_CUDA(cudaFuncSetAttribute(imma_q4k_fold_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IMMA_SMEM));
  if ((rc = init_np<ConvQ8_0, DrainBlockScaled>()) != XNQ_OK) return rc;
  if ((rc = init_np<ConvQ4_0, DrainBlockScaled>()) != XNQ_OK) return rc;
  unsigned int zero = 0;
  XNQ_CUDA(cudaMemcpyToSymbol(g_imma_status, &zero, sizeof(zero)));
  return XNQ_OK;
}

#ifdef XNQ_DEV_TRACE
extern "C" int xnq_dev_imma_trace(long long *out) { return cudaMemcpyFromSymbol(out, g_imma_trace, sizeof(long long) * 32) == cudaSuccess ? 0 : -6; }
extern "C" int xnq_dev_imma_timeline(long long *out) { return cudaMemcpyFromSymbol(out, g_imma_tl, sizeof(long long) * 8 * 64) == cudaSuccess ? 0 : -6; }
#endif

void imma_set_fold(int on) { g_fold.store(on); }

int imma_status(unsigned int *bits) {
  XNQ_CUDA(cudaMemcpyFromSymbol(bits, g_imma_status, sizeof(*bits)));
  return XNQ_OK;
}

} // namespace xnq
