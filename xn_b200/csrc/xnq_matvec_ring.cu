// Decode matvec, m == 1: persistent ring kernel, a few large bulk copies per CTA.
//
// One CTA per SM owns a contiguous band of weight rows and streams it through (almost) all of the SM's
// shared memory, so that the bytes in flight cover HBM's bandwidth x latency (well over 100 KB per SM).
// A stage of the ring holds a run of adjacent weight rows, i.e. one contiguous run of global memory per
// stream, which one producer lane requests with one 1-D bulk-async copy per stream (cp.async.bulk, the
// non-tensor form of TMA; never multicast) that completes on the stage's mbarrier. The copy engine takes
// some 60 ns per copy whatever its size (measured: one copy per row, or per pair of rows, made the issue of
// the copies the bottleneck), so stages are as large as two of them still fit. Sixteen consumer warps take
// one or two rows of a stage each, run the dots against activations they keep in registers, reduce with
// shuffles and store.
//
// The activation row is quantized in the prologue (same device function, same bytes as the stand-alone
// quantizer; the reference's quantize_lhs, k_quants.rs:2015-2026) into a shared-memory image whose
// 16-byte chunks are XOR-swizzled, so that the strided reads with which every lane then loads ITS
// slices of the int8 activations, block scales and block sums into registers are free of bank
// conflicts (unswizzled, those reads were eight-way conflicts and cost over 2 us per launch). A lane
// works on the same k positions of every row, so the main loop reads shared memory only for weights.
//
// k above 4096: a warp keeps at most 4096 activations in registers, so KS = ceil(k / 4096) warps (rounded
// up to a power of two) share a row, each on its own segment of k; stages still hold whole rows. The
// segments' partial sums meet in shared memory behind a named barrier and are added in segment order by
// the first warp, so the result does not depend on timing. Those launches take the activations as an
// activation image (quantized by the caller or by the stand-alone quantizer into the workspace).
//
// Launch overlap: the kernel is launched with programmatic stream serialization. CTAs of the next launch
// in the stream take an SM as soon as this launch's CTA there has left and their producer requests the
// first stages at once (weights are immutable after upload); x is read and y written only after
// griddepcontrol.wait, so results are ordered exactly as without the overlap. The producer too executes
// griddepcontrol.wait before its first wait for a stage to be handed back: its consumers cannot hand
// anything back before the previous kernel has retired, and a bounded wait must not count that time.
// A caller that knows which weight the stream will multiply next can say so (xnq_hint_next_weight): the
// kernel then asks for that weight's bytes to be brought into L2 while it streams its own.
//
// GATHER variant (N-sharded weights): results go to this rank's slot of the gathered output, each CTA
// then sweeps its run of results to every peer's slot with coalesced stores, and the last CTA
// publishes this rank's epoch (xnq_comm.cu).
//
// The dot arithmetic is that of xnq_matvec.cu (exact integer block sums, f32 scales, f32
// accumulate; k_quants.rs:287-304, 677-691, 1337-1416, 1743-1799).
//
// Every mbarrier wait is bounded: on expiry the thread records a status bit, stops computing (consumer
// warps keep taking part in the barriers their partners wait on) and the kernel ends; the producer still
// waits (bounded) for the copies it has in flight before it returns. Every bulk copy and every store is
// range-checked first; a refused access is recorded, not made.
#include <algorithm>
#include <cstring>

#include "xnq_common.cuh"
#include "xnq_quantize_act.cuh"
#include "xnq_unpack.cuh"

namespace xnq {

__device__ unsigned int g_matvec_status; // sticky bits: 1 = a consumer's bounded mbarrier wait expired, 2 = the producer's, 4 = a self-check refused an out-of-range copy or store
__device__ unsigned long long g_matvec_check[8]; // first refused access: code, block, iteration, offset, bytes, limit

#ifdef XNQ_DEV_TRACE
__device__ unsigned long long g_matvec_trace[64][16]; // development builds only: %globaltimer at a few points of block 0 and of the last block
__device__ unsigned int g_matvec_trace_n;
#endif

namespace {

constexpr int CW = 16;               // consumer warps per CTA (a power of two)
constexpr int NTHREADS = (CW + 1) * 32; // + one producer warp
constexpr int MAX_R = 2;             // weight rows per consumer warp and stage: 2 where at least two such stages fit, else 1
constexpr int MAX_STAGES = 8;
#ifndef XNQ_MV_EARLY
#define XNQ_MV_EARLY 1
#endif
constexpr int EARLY_STAGES = XNQ_MV_EARLY; // stages requested before the consumers have their activations
constexpr int SEG_UNITS = 16;        // 256-element units of k one warp keeps in registers
constexpr size_t SMEM_BUDGET = 225 * 1024; // one CTA per SM
constexpr uint32_t HINT_CHUNK = 16384;    // bytes per L2 prefetch request for the next weight

struct Ring {
  int nstreams;
  const uint8_t *src[4];   // stream base in global memory (256-byte aligned)
  uint32_t row_bytes[4];   // bytes of one weight row in stream s (multiple of 16)
  uint32_t unit_bytes[4];  // bytes of one 256-element unit of a row in stream s; 0: the stream is read whole by every segment
  uint32_t stream_off[4];  // offset of stream s inside a stage
  uint32_t stage_bytes;    // multiple of 128
  uint32_t row_bytes_total;
  int stage_rows;          // rows per stage = (CW / ks) * rows per warp
  int rows_per_warp;       // 1 or 2
  int nstages;
  int ks;                  // warps (k segments) per row; a power of two that divides CW
  int ks_shift;            // log2(ks)
  // rows of CTA b: rows_q + (b < rows_r), starting at b * rows_q + min(b, rows_r); niter_q = ceil(rows_q / stage_rows) and
  // niter_q1 = ceil((rows_q + 1) / stage_rows) ring passes (set at launch: the kernel divides by nothing at run time, a
  // 64-bit division costs every thread several hundred cycles before the first copy can be issued)
  int rows_q, rows_r, niter_q, niter_q1;
  int seg_units;           // 256-element units per segment (the last segment may hold fewer)
  int nunits;              // units per row = ceil(k / 256)
  uint32_t act_off, part_off, ring_off; // byte offsets in dynamic shared memory
  uint32_t smem_bytes;
  const uint8_t *hint_base; // the weight the stream multiplies next (may be null): asked into L2
  unsigned long long hint_bytes, hint_share;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait of one thread: false (and a sticky status bit) if the phase never completes
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
  atomicOr(&g_matvec_status, bit);
  return false;
}
// bounded wait of a whole warp: lane 0 polls, the other lanes park on the warp barrier
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, 1u) ? 1 : 0;
  __syncwarp();
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// Self-check: record the first out-of-range access instead of performing it.
__device__ __noinline__ void record_violation(unsigned long long code, unsigned long long a, unsigned long long b, unsigned long long c,
                                              unsigned long long d) {
  if ((atomicOr(&g_matvec_status, 4u) & 4u) == 0) {
    g_matvec_check[0] = code;
    g_matvec_check[1] = blockIdx.x;
    g_matvec_check[2] = a;
    g_matvec_check[3] = b;
    g_matvec_check[4] = c;
    g_matvec_check[5] = d;
  }
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
__device__ __forceinline__ float lds_half(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ void named_barrier(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

__device__ __forceinline__ int dot16(const uint4 &w, const int4 &a, int acc) {
  acc = __dp4a((int)w.x, a.x, acc);
  acc = __dp4a((int)w.y, a.y, acc);
  acc = __dp4a((int)w.z, a.z, acc);
  acc = __dp4a((int)w.w, a.w, acc);
  return acc;
}
// unsigned weight bytes x signed activation bytes
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dot16_us(const uint4 &w, const int4 &a, int acc) {
  acc = dp4a_us(w.x, a.x, acc);
  acc = dp4a_us(w.y, a.y, acc);
  acc = dp4a_us(w.z, a.z, acc);
  acc = dp4a_us(w.w, a.w, acc);
  return acc;
}
__device__ __forceinline__ uint4 and4(const uint4 &v, uint32_t m) { return make_uint4(v.x & m, v.y & m, v.z & m, v.w & m); }
__device__ __forceinline__ uint4 shr4(const uint4 &v, int s) { return make_uint4(v.x >> s, v.y >> s, v.z >> s, v.w >> s); }
__device__ __forceinline__ uint4 shl4(const uint4 &v, int s) { return make_uint4(v.x << s, v.y << s, v.z << s, v.w << s); }
__device__ __forceinline__ uint4 or4(const uint4 &a, const uint4 &b) { return make_uint4(a.x | b.x, a.y | b.y, a.z | b.z, a.w | b.w); }

// Position of 16-byte chunk c of the quantized activation row inside its shared-memory image. The lanes
// of a warp read chunks that lie 2, 4, 8 or 16 chunks apart; folding bits 3..5 of the chunk index into
// its low three bits spreads those reads over all banks.
__device__ __forceinline__ int swz(int c) { return c ^ ((c >> 3) & 7); }
__device__ __forceinline__ int4 act16(const int8_t *sq, int chunk) { return *reinterpret_cast<const int4 *>(sq + swz(chunk) * 16); }

// ---- per-format lane state (activations in registers) and row dots ----------------------------------
// sq / sd / sb: the CTA's quantized activation row in shared memory (swizzled codes, block scales, 16-sums).
// u0 / nu: first 256-element unit of the warp's k segment and the number of units in it (nu <= 16).
// row[r][s]: shared-memory address of row r of the warp's slot in stream s, which holds the segment's bytes.
// dot leaves this lane's partial sums of the two row segments in acc.

struct Q4_0Lane { // lane owns blocks lane, lane+32, ... of the segment (4 of them at most)
  static constexpr int NIT = 4;
  int4 alo[NIT], ahi[NIT];
  float da[NIT];
  int bsum8[NIT]; // 8 * sum of the block's 32 activation codes (weights are stored +8)
  int nblk;       // blocks in the segment
  __device__ __forceinline__ void load(const int8_t *sq, const float *sd, const int16_t *sb, int lane, int u0, int nu, int64_t k) {
    const int b0 = u0 * 8;
    nblk = min(nu * 8, (int)(k / QK) - b0);
#pragma unroll
    for (int it = 0; it < NIT; it++) {
      const int b = lane + 32 * it;
      if (b < nblk) {
        alo[it] = act16(sq, 2 * (b0 + b));
        ahi[it] = act16(sq, 2 * (b0 + b) + 1);
        da[it] = sd[b0 + b];
        bsum8[it] = 8 * ((int)sb[2 * (b0 + b)] + (int)sb[2 * (b0 + b) + 1]);
      } else {
        alo[it] = ahi[it] = make_int4(0, 0, 0, 0);
        da[it] = 0.f;
        bsum8[it] = 0;
      }
    }
  }
  template <int R>
  __device__ __forceinline__ void dot(const uint32_t (&row)[R][4], int lane, int, float (&acc)[R]) const {
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; it++) {
      const int b = lane + 32 * it;
      if (b < nblk) {
        uint4 q[R];
        float dw[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
          q[r] = lds128(row[r][0] + b * 16);
          dw[r] = lds_half(row[r][1] + b * 2);
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
          const int s_lo = dot16(and4(q[r], 0x0f0f0f0fu), alo[it], -bsum8[it]);
          const int s_hi = dot16_us(and4(q[r], 0xf0f0f0f0u), ahi[it], 0); // 16 x the high-nibble sum
          acc[r] += (float)(s_lo + (s_hi >> 4)) * dw[r] * da[it];
        }
      }
    }
  }
};

struct Q8_0Lane { // lane owns 16-byte chunks lane, lane+32, ... of the segment (8 of them at most)
  static constexpr int NIT = 8;
  int4 a[NIT];
  float da[NIT];
  int nch;
  __device__ __forceinline__ void load(const int8_t *sq, const float *sd, const int16_t *, int lane, int u0, int nu, int64_t k) {
    const int c0 = u0 * 16;
    nch = min(nu * 16, (int)(k / 16) - c0);
#pragma unroll
    for (int it = 0; it < NIT; it++) {
      const int c = lane + 32 * it;
      if (c < nch) {
        a[it] = act16(sq, c0 + c);
        da[it] = sd[(c0 + c) >> 1];
      } else {
        a[it] = make_int4(0, 0, 0, 0);
        da[it] = 0.f;
      }
    }
  }
  template <int R>
  __device__ __forceinline__ void dot(const uint32_t (&row)[R][4], int lane, int, float (&acc)[R]) const {
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; it++) {
      const int c = lane + 32 * it;
      if (c < nch) {
#pragma unroll
        for (int r = 0; r < R; r++) {
          const uint4 q = lds128(row[r][0] + c * 16);
          const float dw = lds_half(row[r][1] + (c >> 1) * 2);
          acc[r] += (float)dot16(q, a[it], 0) * dw * da[it];
        }
      }
    }
  }
};

struct Q4KLane { // 2 lanes per super-block: lane = 2*s + h; half h owns sub-blocks 4h..4h+3 (qs bytes 64h..64h+63)
  int4 alo[2][2], ahi[2][2]; // [group g' of the half][16-element half of the sub-block]
  int bs_lo[2], bs_hi[2];    // sums of the 32 activation codes under sub-blocks 2g (low nibbles) and 2g+1 (high)
  float da;
  int nsb;
  __device__ __forceinline__ void load(const int8_t *sq, const float *sd, const int16_t *sb, int lane, int u0, int nu, int64_t) {
    nsb = nu;
    const int s = lane >> 1, h = lane & 1;
    if (s < nsb) {
      const int c0 = (u0 + s) * 16 + 8 * h; // first 16-byte chunk (= first 16-sum) of the half
#pragma unroll
      for (int g = 0; g < 2; g++) {
        alo[g][0] = act16(sq, c0 + 4 * g);
        alo[g][1] = act16(sq, c0 + 4 * g + 1);
        ahi[g][0] = act16(sq, c0 + 4 * g + 2);
        ahi[g][1] = act16(sq, c0 + 4 * g + 3);
        const int16_t *b = sb + c0 + 4 * g;
        bs_lo[g] = (int)b[0] + (int)b[1];
        bs_hi[g] = (int)b[2] + (int)b[3];
      }
      da = sd[u0 + s];
    } else {
#pragma unroll
      for (int g = 0; g < 2; g++) {
        alo[g][0] = alo[g][1] = ahi[g][0] = ahi[g][1] = make_int4(0, 0, 0, 0);
        bs_lo[g] = bs_hi[g] = 0;
      }
      da = 0.f;
    }
  }
  template <int R>
  __device__ __forceinline__ void dot(const uint32_t (&row)[R][4], int lane, int, float (&acc)[R]) const {
    const int s = lane >> 1, h = lane & 1;
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
    if (s >= nsb) return;
    uint4 hdr[R], q[R][4];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const uint32_t blk = row[r][0] + s * 144;
      hdr[r] = lds128(blk);
#pragma unroll
      for (int c = 0; c < 4; c++) q[r][c] = lds128(blk + 16 + 64 * h + 16 * c);
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
      const __half2 dm = *reinterpret_cast<const __half2 *>(&hdr[r].x);
      // the half's two 24-bit scale fields: bits [48h, 48h+48) of the 96-bit field array
      const uint32_t lo32 = h ? __funnelshift_r(hdr[r].z, hdr[r].w, 16) : hdr[r].y;
      const uint32_t hi16 = h ? (hdr[r].w >> 16) : (hdr[r].z & 0xffffu);
      const uint32_t f[2] = {lo32 & 0xffffffu, __funnelshift_r(lo32, hi16, 24) & 0xffffffu};
      int t1 = 0, t2 = 0;
#pragma unroll
      for (int g = 0; g < 2; g++) {
        int s_lo = dot16(and4(q[r][2 * g], 0x0f0f0f0fu), alo[g][0], 0);
        s_lo = dot16(and4(q[r][2 * g + 1], 0x0f0f0f0fu), alo[g][1], s_lo);
        // high nibbles stay in place (value * 16, unsigned bytes): one shift per sub-block instead of one per word
        int s_hi = dot16_us(and4(q[r][2 * g], 0xf0f0f0f0u), ahi[g][0], 0);
        s_hi = dot16_us(and4(q[r][2 * g + 1], 0xf0f0f0f0u), ahi[g][1], s_hi);
        t1 += (int)(f[g] & 63) * s_lo + (int)((f[g] >> 6) & 63) * (s_hi >> 4);
        t2 += (int)((f[g] >> 12) & 63) * bs_lo[g] + (int)(f[g] >> 18) * bs_hi[g];
      }
      acc[r] = da * (__low2float(dm) * (float)t1 - __high2float(dm) * (float)t2);
    }
  }
};

struct Q6KLane { // 4 lanes per super-block; lane owns (half h, l-half lh) of super-blocks lane/4, lane/4+8 of the segment
  static constexpr int NIT = 2;
  int4 a[NIT][4];
  int bs32[NIT][4]; // 32 * sum of the group's 16 activation codes (weights are stored +32)
  float da[NIT];
  int nsb;
  __device__ __forceinline__ void load(const int8_t *sq, const float *sd, const int16_t *sb, int lane, int u0, int nu, int64_t) {
    nsb = nu;
    const int u = lane & 3, h = u >> 1, lh = u & 1;
#pragma unroll
    for (int it = 0; it < NIT; it++) {
      const int s = (lane >> 2) + 8 * it;
      if (s < nsb) {
        const int c0 = (u0 + s) * 16 + 8 * h + lh;
#pragma unroll
        for (int gg = 0; gg < 4; gg++) {
          a[it][gg] = act16(sq, c0 + 2 * gg);
          bs32[it][gg] = 32 * (int)sb[c0 + 2 * gg];
        }
        da[it] = sd[u0 + s];
      } else {
#pragma unroll
        for (int gg = 0; gg < 4; gg++) {
          a[it][gg] = make_int4(0, 0, 0, 0);
          bs32[it][gg] = 0;
        }
        da[it] = 0.f;
      }
    }
  }
  // the f16 super-block scales are a small stream that every segment's slot holds whole: index u0 + s there
  template <int R>
  __device__ __forceinline__ void dot(const uint32_t (&row)[R][4], int lane, int u0, float (&acc)[R]) const {
    const int u = lane & 3, h = u >> 1, lh = u & 1;
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; it++) {
      const int s = (lane >> 2) + 8 * it;
      if (s < nsb) {
#pragma unroll
        for (int r = 0; r < R; r++) {
          const uint4 qa = lds128(row[r][0] + s * 128 + 64 * h + 16 * lh);
          const uint4 qb = lds128(row[r][0] + s * 128 + 64 * h + 32 + 16 * lh);
          const uint4 qh = lds128(row[r][1] + s * 64 + 32 * h + 16 * lh);
          const uint2 scw = lds64(row[r][2] + s * 16 + 8 * h);
          const float dw = lds_half(row[r][3] + (u0 + s) * 2);
          uint4 code[4]; // 6-bit codes 0..63 of the four 16-element groups (k_quants.rs:1763-1770)
          code[0] = or4(and4(qa, 0x0f0f0f0fu), and4(shl4(qh, 4), 0x30303030u));
          code[1] = or4(and4(qb, 0x0f0f0f0fu), and4(shl4(qh, 2), 0x30303030u));
          code[2] = or4(and4(shr4(qa, 4), 0x0f0f0f0fu), and4(qh, 0x30303030u));
          code[3] = or4(and4(shr4(qb, 4), 0x0f0f0f0fu), and4(shr4(qh, 2), 0x30303030u));
          const uint64_t sc64 = (((uint64_t)scw.y << 32) | scw.x) >> (8 * lh); // scale of group gg now at byte 2*gg
          int t = 0;
#pragma unroll
          for (int gg = 0; gg < 4; gg++) {
            const int sc = (int)(int8_t)((sc64 >> (16 * gg)) & 0xff);
            t += sc * dot16(code[gg], a[it][gg], -bs32[it][gg]);
          }
          acc[r] += (dw * da[it]) * (float)t;
        }
      }
    }
  }
};

// Quantize the activation row (k <= 4096) into the swizzled shared-memory image, in two steps so that the
// caller can put other memory requests between the loads of x and the arithmetic: the row costs one round trip
// and its loads are not queued behind the bulk copies of the weights.
struct RowLoad {
  static constexpr int PASSES = (4096 / 8 + CW * 32 - 1) / (CW * 32); // consumer threads only
  float v[PASSES][8];
  __device__ __forceinline__ void issue(const void *x, int x_dtype, int64_t k) {
    const int per_row = (int)(k / 8);
#pragma unroll
    for (int p = 0; p < PASSES; p++) {
      const int t = p * CW * 32 + threadIdx.x;
      if (t < per_row) {
        if (x_dtype == XNQ_F32) load8(static_cast<const float *>(x) + (int64_t)t * 8, v[p]);
        else if (x_dtype == XNQ_F16) load8(static_cast<const __half *>(x) + (int64_t)t * 8, v[p]);
        else load8(static_cast<const __nv_bfloat16 *>(x) + (int64_t)t * 8, v[p]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[p][i] = 0.f;
      }
    }
  }
  // returns once the loads of issue() have arrived (a use of every load's result)
  __device__ __forceinline__ void landed() const {
    float s = 0.f;
#pragma unroll
    for (int p = 0; p < PASSES; p++) s += v[p][0] + v[p][4];
    asm volatile("" ::"f"(s) : "memory");
  }
  template <int ACT>
  __device__ __forceinline__ void finish(int64_t k, int8_t *sq, float *sd, int16_t *sb) const {
    const int lane = threadIdx.x & 31;
    const int per_row = (int)(k / 8);
#pragma unroll
    for (int p = 0; p < PASSES; p++) {
      const int t = p * CW * 32 + threadIdx.x;
      if (p * CW * 32 + (int)(threadIdx.x & ~31u) >= per_row) continue; // whole warps skip together
      const Quant8 q = ACT == XNQ_Q8_0 ? quantize8_q8_0(v[p], lane) : quantize8_q8k(v[p], lane);
      if (t < per_row) {
        *reinterpret_cast<uint2 *>(sq + swz(t >> 1) * 16 + (t & 1) * 8) = make_uint2(q.lo, q.hi);
        if (ACT == XNQ_Q8_0) {
          if ((lane & 3) == 0) sd[t / 4] = q.d;
        } else {
          if (lane == 0) sd[t / 32] = q.d;
        }
        if ((lane & 1) == 0) sb[t / 2] = (int16_t)q.sum16;
      }
    }
  }
};

__device__ __forceinline__ void store_out(void *y, int y_dtype, int64_t idx, float v) {
  if (y_dtype == XNQ_F32) static_cast<float *>(y)[idx] = v;
  else if (y_dtype == XNQ_F16) static_cast<__half *>(y)[idx] = __float2half_rn(v);
  else static_cast<__nv_bfloat16 *>(y)[idx] = __float2bfloat16_rn(v);
}

#ifdef XNQ_DEV_TRACE
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define XNQ_TRACE_POINT(i) do { if (tr && threadIdx.x == 0) g_matvec_trace[trace_slot][tb + (i)] = gtime(); } while (0)
#else
#define XNQ_TRACE_POINT(i) do { } while (0)
#endif

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 15, %0;" ::"n"(CW * 32) : "memory"); }

// GATHER: this rank holds rows [col0, col0 + n) of an N-sharded weight; every result goes straight
// into the gathered output of every rank (plain stores through peer mappings), and the last CTA to
// finish publishes this rank's next epoch to every peer.
template <typename LaneT, int ACT, int R, bool GATHER>
__global__ void __launch_bounds__(NTHREADS, 1)
matvec_ring_kernel(WeightView w, const void *x, int x_dtype, void *y, int y_dtype, Ring ring, GatherArgs g, NormArgs na) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t full0 = smem_u32(smem), empty0 = full0 + 8 * MAX_STAGES; // full[MAX_STAGES], empty[MAX_STAGES]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t k = w.k;
  const bool extra_row = (int)blockIdx.x < ring.rows_r;
  const int nrows = ring.rows_q + (extra_row ? 1 : 0);
  const int64_t row_begin = (int64_t)blockIdx.x * ring.rows_q + min((int)blockIdx.x, ring.rows_r);
  const int KS = ring.ks, S = ring.nstages, RPS = ring.stage_rows;
  const int niter = extra_row ? ring.niter_q1 : ring.niter_q;
  const uint32_t ring0 = smem_u32(smem + ring.ring_off);
#ifdef XNQ_DEV_TRACE
  __shared__ unsigned int trace_slot;
  const bool tr = blockIdx.x == 0 || blockIdx.x == gridDim.x - 1;
  const int tb = blockIdx.x == 0 ? 0 : 8;
  if (tr && threadIdx.x == 0) {
    if (blockIdx.x == 0) trace_slot = atomicAdd(&g_matvec_trace_n, 1u) & 63;
    else trace_slot = g_matvec_trace_n & 63;
    g_matvec_trace[trace_slot][tb + 0] = gtime();
  }
#endif
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, CW); // one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents(); // the next launch in the stream may start as soon as SMs are free

  if (warp == CW) { // ---- producer: weights are immutable after upload, no dependency on earlier kernels ----
    int issued = 0;
    bool dead = false, synced = false;
    int s = -1;
    uint32_t ph = 0; // stage it % S and (it / S) & 1, kept as counters
    for (int it = 0; it < niter; it++) {
      if (++s == S) s = 0, ph ^= 1u;
      // The first stages are requested at once. The rest of the ring is requested only when the consumers have their
      // activations: requested earlier, its bytes sit in the memory system's queues in front of the loads of x, which
      // every consumer needs before it can start (measured: x then takes 1 to 3 us instead of half a microsecond), and
      // those stages are not consumed before the first ones anyway.
      if (it == EARLY_STAGES) {
        asm volatile("bar.sync 14, %0;" ::"n"(NTHREADS) : "memory"); // all 32 lanes: the barrier counts threads
        synced = true;
      }
      if (lane == 0 && !dead) {
        if (it == S) pdl_wait(); // nothing is handed back before the previous kernel has retired: do not count that time
        if (it >= S && !mbar_wait(empty0 + 8 * s, ph ^ 1u, 2u)) {
          dead = true;
          continue;
        }
        const int rows = min(RPS, nrows - it * RPS);
        issued = it + 1;
        mbar_expect_tx(full0 + 8 * s, (uint32_t)rows * ring.row_bytes_total);
#pragma unroll
        for (int st = 0; st < 4; st++) {
          if (st < ring.nstreams) {
            const unsigned long long off = (unsigned long long)(row_begin + (int64_t)it * RPS) * ring.row_bytes[st];
            const unsigned long long bytes = (unsigned long long)rows * ring.row_bytes[st];
            const unsigned long long limit = (unsigned long long)w.n * ring.row_bytes[st];
            const uint32_t dst_off = ring.ring_off + s * ring.stage_bytes + ring.stream_off[st];
            if (off + bytes > limit || (bytes & 15) || (off & 15) || (dst_off & 15) || dst_off + bytes > ring.smem_bytes ||
                ((unsigned long long)ring.src[st] & 15)) {
              record_violation(0x100 + st, it, off, bytes, limit);
              continue; // the stage never completes; consumers give up on their bounded wait
            }
            bulk_g2s(ring0 + s * ring.stage_bytes + ring.stream_off[st], ring.src[st] + off, (uint32_t)bytes, full0 + 8 * s);
          }
        }
      }
    }
    if (!synced) asm volatile("bar.sync 14, %0;" ::"n"(NTHREADS) : "memory"); // the consumers arrive on it in any case
    if (lane == 0) {
      // The weight this stream multiplies next, if the caller named it: this CTA's share is asked into L2 now that
      // all of the CTA's own rows have been requested, so the requests fill the memory system while the consumers
      // finish (asked for earlier, they compete with the CTA's own stream and slow it down).
      if (ring.hint_base && issued == niter) {
        const unsigned long long share = ring.hint_share; // hint_bytes / grid, rounded up to whole chunks
        const unsigned long long h0 = share * blockIdx.x, h1 = min(h0 + share, ring.hint_bytes & ~15ull);
        for (unsigned long long o = h0; o < h1; o += HINT_CHUNK) bulk_prefetch_l2(ring.hint_base + o, (uint32_t)min((unsigned long long)HINT_CHUNK, h1 - o));
      }
      // nothing may be in flight into this CTA's shared memory when it exits
      for (int it = max(0, issued - S); it < issued; it++) mbar_wait(full0 + 8 * (it % S), (it / S) & 1, 2u);
    }
    return;
  }

  // ---- consumers ----
  const int rl = warp >> ring.ks_shift, seg = warp - rl * KS;
  const int u0 = seg * ring.seg_units; // first unit of this warp's segment
  const int nu = min(ring.seg_units, ring.nunits - u0);
  pdl_wait(); // x may be the previous kernel's output; y may still be read by it
  XNQ_TRACE_POINT(1);
  int8_t *sq = reinterpret_cast<int8_t *>(smem + ring.act_off);
  const int act_blk = ACT == XNQ_Q8_0 ? QK : QK_K;
  const int nblk = (int)(k / act_blk);
  float *sd = reinterpret_cast<float *>(sq + ((k + 127) & ~(int64_t)127)); // the swizzle permutes chunks inside aligned groups of eight
  int16_t *sb = reinterpret_cast<int16_t *>(reinterpret_cast<unsigned char *>(sd) + ((nblk * 4 + 15) & ~15));
  bool told = false; // whether the producer has been told that the activations are here
  if (x_dtype == XNQ_ACT_IMAGE) {
    // activations quantized ahead of the call: copy the row's image (codes | block scales | 16-sums, each
    // section 256-byte aligned), swizzling the code chunks on the way
    const unsigned char *img = static_cast<const unsigned char *>(x);
    const unsigned char *img_d = img + ((k + 255) & ~(int64_t)255);
    const unsigned char *img_b = img_d + (((int64_t)nblk * 4 + 255) & ~(int64_t)255);
    for (int i = threadIdx.x; i < k / 16; i += CW * 32) reinterpret_cast<uint4 *>(sq)[swz(i)] = reinterpret_cast<const uint4 *>(img)[i];
    for (int i = threadIdx.x; i < nblk; i += CW * 32) sd[i] = reinterpret_cast<const float *>(img_d)[i];
    for (int i = threadIdx.x; i < k / 32; i += CW * 32) reinterpret_cast<uint32_t *>(sb)[i] = reinterpret_cast<const uint32_t *>(img_b)[i];
  } else if (na.x_in) {
    // Residual add + RMSNorm of the row, then the quantizer: the arithmetic, and the order of the sum of squares, of the
    // stand-alone add+RMSNorm kernel (one run of 8 per thread, one 256-element partial sum per warp, partial sums added in
    // index order), so the image is the one that kernel would have written.
    static_assert(RowLoad::PASSES == 1, "one run of 8 elements per consumer thread");
    RowLoad xr;
    float gw[8];
    const int per_row = (int)(k / 8), t = threadIdx.x;
    const bool valid = t < per_row;
    if (valid) {
      load8(na.x_in + (int64_t)t * 8, xr.v[0]);
      load8(na.weight + (int64_t)t * 8, gw);
    }
    if (na.wait_ctl) { // the summands come from the peers: await their epochs (lane p awaits rank p), then let the CTA read them
      if (warp == 0 && lane < na.wait_world && lane != na.wait_rank && na.wait_ctl[3] == 0) {
        const unsigned int epoch = na.wait_ctl[0];
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
          unsigned int v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(na.wait_row + lane) : "memory");
          if ((int)(v - epoch) >= 0) break;
          unsigned long long t1;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
          if (t1 - t0 > GATHER_WAIT_LIMIT_NS) { // a late peer is reported once and not awaited again
            atomicOr(na.wait_ctl + 3, 1u << lane);
            break;
          }
        }
      }
      consumer_sync();
    }
    if (valid) {
      for (int q = 0; q < na.parts; q++) {
        float a[8];
        load8(na.delta + (int64_t)q * k + (int64_t)t * 8, a);
#pragma unroll
        for (int e = 0; e < 8; e++) xr.v[0][e] = __fadd_rn(xr.v[0][e], a[e]);
      }
      if (blockIdx.x == 0) {
        *reinterpret_cast<float4 *>(na.x_out + (int64_t)t * 8) = make_float4(xr.v[0][0], xr.v[0][1], xr.v[0][2], xr.v[0][3]);
        *reinterpret_cast<float4 *>(na.x_out + (int64_t)t * 8 + 4) = make_float4(xr.v[0][4], xr.v[0][5], xr.v[0][6], xr.v[0][7]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) xr.v[0][e] = 0.f, gw[e] = 0.f;
    }
    xr.landed(); // the row and its summands are here: the rest of the ring may be requested while the norm is computed
    asm volatile("bar.arrive 14, %0;" ::"n"(NTHREADS) : "memory");
    told = true;
    float *red = reinterpret_cast<float *>(smem + ring.part_off); // free until the first stage is multiplied
    const int np = (int)((k + 255) / 256);
    if (warp < np) {
      const float s = rms_warp_sum(valid ? rms_run_sum(xr.v[0]) : 0.f);
      if (lane == 0) red[warp] = s;
    }
    consumer_sync();
    float tot = 0.f;
    for (int i = 0; i < np; i++) tot += red[i];
    const float r = rms_scale(tot, (int)k, na.eps);
#pragma unroll
    for (int e = 0; e < 8; e++) xr.v[0][e] = rms_apply(xr.v[0][e], r, gw[e]);
    consumer_sync(); // every warp has read the partial sums: the scratch may be reused
    xr.template finish<ACT>(k, sq, sd, sb);
  } else {
    RowLoad xr;
    xr.issue(x, x_dtype, k);
    xr.landed();
    asm volatile("bar.arrive 14, %0;" ::"n"(NTHREADS) : "memory"); // the row is here: the rest of the ring may be requested while it is quantized
    told = true;
    xr.template finish<ACT>(k, sq, sd, sb);
  }
  if (!told) asm volatile("bar.arrive 14, %0;" ::"n"(NTHREADS) : "memory"); // the producer may request the rest of the ring
  consumer_sync();
  XNQ_TRACE_POINT(2);
  LaneT st;
  st.load(sq, sd, sb, lane, u0, nu, k);
  XNQ_TRACE_POINT(3);
  float *parts = reinterpret_cast<float *>(smem + ring.part_off); // [2][CW][MAX_R] segment sums (KS > 1)
  // where this warp's segment starts inside a row of each stream (streams with unit_bytes 0 are read whole)
  uint32_t seg_off[4];
#pragma unroll
  for (int q = 0; q < 4; q++) seg_off[q] = (uint32_t)u0 * ring.unit_bytes[q];

  bool alive = true;
  int s = -1;
  uint32_t ph = 0; // stage it % S and (it / S) & 1
  for (int it = 0; it < niter; it++) {
    if (++s == S) s = 0, ph ^= 1u;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
    if (alive) alive = mbar_wait_warp(full0 + 8 * s, ph);
#ifdef XNQ_DEV_TRACE
    if (it == 0) XNQ_TRACE_POINT(4);
#endif
    const int rows = min(RPS, nrows - it * RPS);
    const int slot0 = rl * R; // this warp's first row inside the stage
    if (alive && slot0 < rows) {
      uint32_t row[R][4];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const int slot = min(slot0 + r, rows - 1); // a duplicate of the last row past the ragged end; never stored
#pragma unroll
        for (int q = 0; q < 4; q++) row[r][q] = ring0 + s * ring.stage_bytes + ring.stream_off[q] + (uint32_t)slot * ring.row_bytes[q] + seg_off[q];
      }
      st.template dot<R>(row, lane, u0, acc);
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
        for (int r = 0; r < R; r++) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s); // dead or alive: the producer must not wait for a warp that gave up
    float v = acc[0]; // lane r stores row r of the warp's rows
#pragma unroll
    for (int r = 1; r < R; r++) v = lane == r ? acc[r] : v;
    if (KS > 1) { // the rows' segment sums meet in shared memory and are added in segment order
      float *part = parts + (it & 1) * CW * MAX_R;
      if (lane < R) part[warp * MAX_R + lane] = v;
      named_barrier(1 + rl, KS * 32); // warps of one row take part in every stage, dead or alive
      if (seg == 0 && lane < R) {
        v = part[warp * MAX_R + lane];
        for (int j = 1; j < KS; j++) v += part[(warp + j) * MAX_R + lane];
      }
    }
    if (seg == 0 && lane < R && slot0 + lane < rows && alive) {
      const int64_t idx = row_begin + (int64_t)it * RPS + slot0 + lane;
      if (idx < 0 || idx >= w.n) record_violation(0x200, it, (unsigned long long)idx, slot0, w.n);
      else if (!GATHER) store_out(y, y_dtype, idx, v);
      else store_out(g.dst[g.rank], y_dtype, g.col0 + idx, v); // the peers get the CTA's whole run of rows in one sweep below
    }
  }
  XNQ_TRACE_POINT(5);
  if (GATHER) {
    consumer_sync(); // the CTA's results are in the local buffer
    // One coalesced sweep of this CTA's contiguous run of results to every peer: 16-byte vectors where
    // the run is aligned, single elements at its ragged ends. (One 4-byte store per row and peer from
    // inside the loop costs a link packet each; at eight ranks that dominated the launch.)
    if (g.world > 1 && nrows > 0) {
      const int es = y_dtype == XNQ_F32 ? 4 : 2;
      const size_t off = (size_t)(g.col0 + row_begin) * es;
      const char *src = static_cast<const char *>(g.dst[g.rank]) + off;
      const int nbytes = nrows * es;
      const int head = min(nbytes, (int)((16 - (reinterpret_cast<uintptr_t>(src) & 15)) & 15));
      const int nvec = (nbytes - head) / 16, tail0 = head + nvec * 16;
      for (int v = threadIdx.x; v < nvec; v += CW * 32) {
        const uint4 val = __ldcg(reinterpret_cast<const uint4 *>(src + head) + v);
        for (int p = 0; p < g.world; p++)
          if (p != g.rank) reinterpret_cast<uint4 *>(static_cast<char *>(g.dst[p]) + off + head)[v] = val;
      }
      const int nedge = (head + (nbytes - tail0)) / es; // elements before the first and after the last full vector
      for (int e = threadIdx.x; e < nedge; e += CW * 32) {
        const int b = e * es < head ? e * es : tail0 + (e * es - head);
        if (es == 4) {
          const uint32_t val = __ldcg(reinterpret_cast<const uint32_t *>(src + b));
          for (int p = 0; p < g.world; p++)
            if (p != g.rank) *reinterpret_cast<uint32_t *>(static_cast<char *>(g.dst[p]) + off + b) = val;
        } else {
          const unsigned short val = __ldcg(reinterpret_cast<const unsigned short *>(src + b));
          for (int p = 0; p < g.world; p++)
            if (p != g.rank) *reinterpret_cast<unsigned short *>(static_cast<char *>(g.dst[p]) + off + b) = val;
        }
      }
      consumer_sync();
    }
    if (threadIdx.x < 32) gather_publish_and_wait(g);
  }
}

int g_num_sms = 0;
thread_local const xnq_weight *t_hint_next = nullptr; // xnq_hint_next_weight: consumed by the next one-row launch of this thread

int plan_ring(const WeightView &w, Ring &r) {
  const int64_t k = w.k;
  std::memset(&r, 0, sizeof(r));
  switch (w.dtype) {
    case XNQ_Q4_0:
      r.nstreams = 2;
      r.row_bytes[0] = (uint32_t)(k / 2); r.src[0] = w.qs; r.unit_bytes[0] = 128;
      r.row_bytes[1] = (uint32_t)(w.dstride * 2); r.src[1] = reinterpret_cast<const uint8_t *>(w.d); r.unit_bytes[1] = 16;
      break;
    case XNQ_Q8_0:
      r.nstreams = 2;
      r.row_bytes[0] = (uint32_t)k; r.src[0] = w.qs; r.unit_bytes[0] = 256;
      r.row_bytes[1] = (uint32_t)(w.dstride * 2); r.src[1] = reinterpret_cast<const uint8_t *>(w.d); r.unit_bytes[1] = 16;
      break;
    case XNQ_Q4K:
      r.nstreams = 1;
      r.row_bytes[0] = (uint32_t)(k / QK_K * 144); r.src[0] = w.qs; r.unit_bytes[0] = 144;
      break;
    case XNQ_Q6K:
      r.nstreams = 4;
      r.row_bytes[0] = (uint32_t)(k / 2); r.src[0] = w.qs; r.unit_bytes[0] = 128;
      r.row_bytes[1] = (uint32_t)(k / 4); r.src[1] = w.qh; r.unit_bytes[1] = 64;
      r.row_bytes[2] = (uint32_t)(k / 16); r.src[2] = reinterpret_cast<const uint8_t *>(w.sc); r.unit_bytes[2] = 16;
      r.row_bytes[3] = (uint32_t)(w.dstride * 2); r.src[3] = reinterpret_cast<const uint8_t *>(w.d); r.unit_bytes[3] = 0; // whole row of f16 scales per slot
      break;
    default: return 0;
  }
  for (int st = 0; st < r.nstreams; st++) {
    if (r.row_bytes[st] % 16) return 0;
    r.row_bytes_total += r.row_bytes[st];
  }
  r.nunits = (int)((k + 255) / 256);
  int ks = 1;
  while (ks * SEG_UNITS < r.nunits) ks *= 2;
  if (ks > CW) return 0;
  if (ks > 1 && (k % 256)) return 0; // segments are cut at 256-element units
  r.ks = ks;
  r.seg_units = (r.nunits + ks - 1) / ks;
  if ((ks - 1) * r.seg_units >= r.nunits) return 0; // every segment must hold at least one unit
  if (ks == 1) r.unit_bytes[0] = r.unit_bytes[1] = r.unit_bytes[2] = r.unit_bytes[3] = 0; // one segment: every stream is read from its start
  const int act_blk = (w.dtype == XNQ_Q4_0 || w.dtype == XNQ_Q8_0) ? QK : QK_K;
  const uint32_t act_bytes = (uint32_t)(((k + 127) & ~(int64_t)127) + ((k / act_blk * 4 + 15) & ~15) + ((k / 16 * 2 + 15) & ~15));
  r.act_off = 2 * MAX_STAGES * 8;
  r.part_off = (r.act_off + act_bytes + 15) & ~15u;
  r.ring_off = (r.part_off + 2 * CW * MAX_R * 4 + 127) & ~127u;
  if (r.ring_off >= SMEM_BUDGET) return 0;
  const size_t avail = SMEM_BUDGET - r.ring_off;
  r.nstages = 0;
  for (int rows = MAX_R; rows >= 1 && r.nstages < 2; rows--) { // two rows per warp where at least three (else two) such stages fit
    r.rows_per_warp = rows;
    r.stage_rows = (CW / ks) * rows;
    uint32_t off = 0;
    for (int st = 0; st < r.nstreams; st++) {
      r.stream_off[st] = off;
      off += (uint32_t)r.stage_rows * r.row_bytes[st];
    }
    r.stage_bytes = (off + 127) & ~127u;
    r.nstages = (int)std::min<size_t>(MAX_STAGES, avail / r.stage_bytes);
    if (rows == MAX_R && r.nstages < 3) r.nstages = 0;
  }
  if (r.nstages < 2) return 0;
  r.smem_bytes = r.ring_off + (uint32_t)r.nstages * r.stage_bytes;
  return ks;
}

template <typename LaneT, int ACT>
int launch_fmt(const WeightView &w, const void *x, int x_dtype, void *y, int y_dtype, const Ring &r, cudaStream_t s, const GatherArgs *g, const NormArgs *norm) {
  const NormArgs na = norm ? *norm : NormArgs{};
  const int64_t max_ctas = (w.n + r.stage_rows - 1) / r.stage_rows; // at least one stage of rows per CTA
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>((int64_t)g_num_sms, max_ctas));
  Ring rr = r;
  rr.rows_q = (int)(w.n / grid), rr.rows_r = (int)(w.n % grid);
  rr.niter_q = (rr.rows_q + r.stage_rows - 1) / r.stage_rows, rr.niter_q1 = (rr.rows_q + r.stage_rows) / r.stage_rows;
  rr.ks_shift = 0;
  while ((1 << rr.ks_shift) < r.ks) rr.ks_shift++;
  rr.hint_share = ((r.hint_bytes / grid) + HINT_CHUNK - 1) & ~(unsigned long long)(HINT_CHUNK - 1);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = r.smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (r.rows_per_warp == 2) {
    if (g) XNQ_CUDA(cudaLaunchKernelEx(&cfg, matvec_ring_kernel<LaneT, ACT, 2, true>, w, x, x_dtype, y, y_dtype, rr, *g, na));
    else XNQ_CUDA(cudaLaunchKernelEx(&cfg, matvec_ring_kernel<LaneT, ACT, 2, false>, w, x, x_dtype, y, y_dtype, rr, GatherArgs{}, na));
  } else {
    if (g) XNQ_CUDA(cudaLaunchKernelEx(&cfg, matvec_ring_kernel<LaneT, ACT, 1, true>, w, x, x_dtype, y, y_dtype, rr, *g, na));
    else XNQ_CUDA(cudaLaunchKernelEx(&cfg, matvec_ring_kernel<LaneT, ACT, 1, false>, w, x, x_dtype, y, y_dtype, rr, GatherArgs{}, na));
  }
  count_launch();
  return XNQ_OK;
}

template <typename LaneT, int ACT>
int init_fmt() {
  XNQ_CUDA(cudaFuncSetAttribute(matvec_ring_kernel<LaneT, ACT, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET));
  XNQ_CUDA(cudaFuncSetAttribute(matvec_ring_kernel<LaneT, ACT, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET));
  XNQ_CUDA(cudaFuncSetAttribute(matvec_ring_kernel<LaneT, ACT, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET));
  XNQ_CUDA(cudaFuncSetAttribute(matvec_ring_kernel<LaneT, ACT, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET));
  return XNQ_OK;
}

} // namespace

bool matvec_tma_supported(const WeightView &w, int64_t m) {
  if (m != 1 || g_num_sms <= 0 || w.n < 1) return false;
  Ring r;
  return plan_ring(w, r) > 0;
}

// The kernel quantizes a float activation row itself only when one warp holds the whole row (k <= 4096);
// longer rows must come as an activation image.
bool matvec_tma_wants_image(const WeightView &w) {
  Ring r;
  return plan_ring(w, r) > 1 || w.k > 4096;
}

void matvec_hint_next(const xnq_weight *w) { t_hint_next = w; }

int launch_matvec_tma(const WeightView &w, const void *x, int x_dtype, void *y, int y_dtype, cudaStream_t s, const GatherArgs *g, const NormArgs *norm) {
  Ring r;
  const int ks = plan_ring(w, r);
  if (!ks) return fail(XNQ_ERR_SIZE, "matvec_ring: no ring fits k = %lld", (long long)w.k);
  if (x_dtype != XNQ_ACT_IMAGE && (ks > 1 || w.k > 4096)) return fail(XNQ_ERR_SIZE, "matvec_ring: k = %lld needs the activations as an image", (long long)w.k);
  if (norm && norm->x_in && (x_dtype == XNQ_ACT_IMAGE || w.k % 8)) return fail(XNQ_ERR_SHAPE, "matvec_ring: the norm prologue takes f32 rows of a multiple of 8 values");
  if (t_hint_next) { // one-shot: the named weight is asked into L2 by this launch
    r.hint_base = static_cast<const uint8_t *>(t_hint_next->base);
    r.hint_bytes = t_hint_next->bytes;
    t_hint_next = nullptr;
  }
  switch (w.dtype) {
    case XNQ_Q4_0: return launch_fmt<Q4_0Lane, XNQ_Q8_0>(w, x, x_dtype, y, y_dtype, r, s, g, norm);
    case XNQ_Q8_0: return launch_fmt<Q8_0Lane, XNQ_Q8_0>(w, x, x_dtype, y, y_dtype, r, s, g, norm);
    case XNQ_Q4K: return launch_fmt<Q4KLane, XNQ_Q8K>(w, x, x_dtype, y, y_dtype, r, s, g, norm);
    case XNQ_Q6K: return launch_fmt<Q6KLane, XNQ_Q8K>(w, x, x_dtype, y, y_dtype, r, s, g, norm);
  }
  return fail(XNQ_ERR_DTYPE, "matvec_ring: dtype %d", w.dtype);
}

int matvec_tma_init(int device) {
  cudaDeviceProp prop;
  XNQ_CUDA(cudaGetDeviceProperties(&prop, device));
  g_num_sms = prop.multiProcessorCount;
  int rc;
  if ((rc = init_fmt<Q4_0Lane, XNQ_Q8_0>()) != XNQ_OK) return rc;
  if ((rc = init_fmt<Q8_0Lane, XNQ_Q8_0>()) != XNQ_OK) return rc;
  if ((rc = init_fmt<Q4KLane, XNQ_Q8K>()) != XNQ_OK) return rc;
  if ((rc = init_fmt<Q6KLane, XNQ_Q8K>()) != XNQ_OK) return rc;
  unsigned int zero = 0;
  XNQ_CUDA(cudaMemcpyToSymbol(g_matvec_status, &zero, sizeof(zero)));
  return XNQ_OK;
}

int matvec_status(unsigned int *bits) {
  XNQ_CUDA(cudaMemcpyFromSymbol(bits, g_matvec_status, sizeof(*bits)));
  return XNQ_OK;
}

int matvec_check_record(unsigned long long out[8]) {
  XNQ_CUDA(cudaMemcpyFromSymbol(out, g_matvec_check, sizeof(unsigned long long) * 8));
  return XNQ_OK;
}

#ifdef XNQ_DEV_TRACE
extern "C" int xnq_dev_matvec_trace(unsigned long long *out, unsigned int *n) {
  if (cudaMemcpyFromSymbol(out, g_matvec_trace, sizeof(unsigned long long) * 64 * 16) != cudaSuccess) return -6;
  if (cudaMemcpyFromSymbol(n, g_matvec_trace_n, sizeof(unsigned int)) != cudaSuccess) return -6;
  return 0;
}
#endif

} // namespace xnq
