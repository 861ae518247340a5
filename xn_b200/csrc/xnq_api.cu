// C ABI of the xnq library: argument validation, weight handles, dispatch. See include/xnq.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <mutex>
#include <new>
#include <vector>

#include "xnq_common.cuh"

namespace xnq {

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { g_err[0] = 0; }

static std::atomic<uint64_t> g_launches{0};
static std::atomic<bool> g_opt_matvec_tma{true};
static std::atomic<int> g_opt_gather_cta_fence{1};
static std::atomic<int> g_opt_host_direct_y{1};
static std::atomic<int> g_opt_matvec_mma{1};
static std::atomic<int> g_opt_imma{1};
static bool use_imma(const xnq_weight *w, int64_t m) { return m >= 2 && m <= IMMA_MAX_M && g_opt_imma.load(std::memory_order_relaxed) && imma_supported(w->v, m); }
// Small batches: the integer-MMA kernel where it serves the weight and wins (Q4_K, five rows and up), else the
// dp4a kernel. Returns the rows per launch.
int64_t small_batch_pass(const xnq_weight *w, int64_t m, int y_dtype, bool *use_mma) {
  const int64_t mp = (m >= 5 && g_opt_matvec_mma.load(std::memory_order_relaxed)) ? matvec_mma_rows_per_pass(w->v, y_dtype) : 0;
  *use_mma = mp > 0;
  return mp > 0 ? mp : matvec_rows_per_pass(w->v.dtype, w->v.k);
}
int gather_cta_fence_scope() { return g_opt_gather_cta_fence.load(std::memory_order_relaxed); }
bool matvec_tma_enabled() { return g_opt_matvec_tma.load(std::memory_order_relaxed); }
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

struct Profile {
  bool on = false;
  std::vector<cudaEvent_t> ev; // start/stop pairs
  size_t used = 0;
};
static thread_local Profile g_prof;
void profile_mark(cudaStream_t s, bool start) {
  Profile &p = g_prof;
  if (!p.on) return;
  if (start) {
    if (p.used + 2 > p.ev.size()) return;
    cudaEventRecord(p.ev[p.used], s);
  } else {
    if (p.used + 2 > p.ev.size()) return;
    cudaEventRecord(p.ev[p.used + 1], s);
    p.used += 2;
  }
}

static inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
static inline size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

// Bytes of the device image of `n` rows, and the sub-buffer offsets inside it.
struct Plan {
  size_t qs, qh, sc, d, total;
  int64_t dstride;
};
static Plan plan_for(int dtype, int64_t n, int64_t k) {
  Plan p{};
  const int64_t nblk = k / block_size(dtype);
  p.dstride = (nblk + 7) & ~(int64_t)7;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off += up256(bytes);
    return at;
  };
  switch (dtype) {
    case XNQ_Q4_0:
      p.qs = take((size_t)n * nblk * 16);
      p.d = take((size_t)n * p.dstride * 2);
      break;
    case XNQ_Q8_0:
      p.qs = take((size_t)n * k);
      p.d = take((size_t)n * p.dstride * 2);
      break;
    case XNQ_Q4K:
      p.qs = take((size_t)n * nblk * 144);
      p.dstride = 0;
      break;
    case XNQ_Q6K:
      p.qs = take((size_t)n * nblk * 128);
      p.qh = take((size_t)n * nblk * 64);
      p.sc = take((size_t)n * nblk * 16);
      p.d = take((size_t)n * p.dstride * 2);
      break;
  }
  p.total = off ? off : 256;
  return p;
}

int check_activations(const char *who, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx) {
  if (!is_float_dtype(x_dtype)) return fail(XNQ_ERR_DTYPE, "%s: activation dtype %d is not f32/f16/bf16", who, x_dtype);
  if (m < 0) return fail(XNQ_ERR_SHAPE, "%s: m = %lld", who, (long long)m);
  if (ldx < k) return fail(XNQ_ERR_SHAPE, "%s: ldx = %lld is smaller than k = %lld", who, (long long)ldx, (long long)k);
  if (m > 0 && !x) return fail(XNQ_ERR_NULL, "%s: x is NULL", who);
  const size_t es = type_size(x_dtype);
  if (m > 0 && (!aligned(x, 16) || (m > 1 && (ldx * es) % 16 != 0)))
    return fail(XNQ_ERR_ALIGN, "%s: activation rows must start 16-byte aligned (x=%p, ldx=%lld)", who, x, (long long)ldx);
  return XNQ_OK;
}

} // namespace xnq

using namespace xnq;

// xnq_matmul_t on activations that were quantized ahead of the call (x_dtype == XNQ_ACT_IMAGE): the decode
// kernels read the image directly; nothing is quantized and no scratch is used.
// activations in the integer tensor-core kernel's own layout (XNQ_ACT_OPERAND): one kernel
static int matmul_from_operand(const xnq_weight *w, const void *image, int64_t m, void *y, int y_dtype, int64_t ldy, void *workspace, size_t ws_bytes,
                               cudaStream_t s) {
  const int64_t k = w->v.k, n = w->v.n;
  if (!is_float_dtype(y_dtype)) return fail(XNQ_ERR_DTYPE, "matmul_t: output dtype %d is not f32/f16/bf16", y_dtype);
  if (ldy < n) return fail(XNQ_ERR_SHAPE, "matmul_t: ldy = %lld is smaller than n = %lld", (long long)ldy, (long long)n);
  if (m == 0 || n == 0) return XNQ_OK;
  if (!image || !y) return fail(XNQ_ERR_NULL, "matmul_t: image or y is NULL");
  if (!aligned(image, 256)) return fail(XNQ_ERR_ALIGN, "matmul_t: the operand image must be 256-byte aligned");
  if (!aligned(y, type_size(y_dtype))) return fail(XNQ_ERR_ALIGN, "matmul_t: y is not aligned to its element size");
  if (act_dtype_for(w->v.dtype) != XNQ_Q8K || !is_fast_dtype(w->v.dtype) || !use_imma(w, m))
    return fail(XNQ_ERR_UNSUPPORTED, "matmul_t: an operand image serves 2..%lld rows on weights of the integer tensor-core kernel with Q8_K activations (dtype %d, m = %lld)",
                (long long)IMMA_MAX_M, w->v.dtype, (long long)m);
  if (!workspace || !aligned(workspace, 256) || ws_bytes < imma_workspace_bytes(m, k, n))
    return fail(XNQ_ERR_SIZE, "matmul_t: the workspace (256-byte aligned, %zu bytes) is needed for the partial sums", imma_workspace_bytes(m, k, n));
  return launch_imma(w->v, image, XNQ_ACT_OPERAND, m, k, y, y_dtype, ldy, workspace, s);
}

static int matmul_from_image(const xnq_weight *w, const void *image, int64_t m, void *y, int y_dtype, int64_t ldy, void *workspace, size_t ws_bytes,
                             cudaStream_t s) {
  const int64_t k = w->v.k, n = w->v.n;
  if (m < 0 || m > MATVEC_MAX_M) return fail(XNQ_ERR_SIZE, "matmul_t: an activation image serves 0..%d rows, m = %lld", MATVEC_MAX_M, (long long)m);
  if (!is_float_dtype(y_dtype)) return fail(XNQ_ERR_DTYPE, "matmul_t: output dtype %d is not f32/f16/bf16", y_dtype);
  if (ldy < n) return fail(XNQ_ERR_SHAPE, "matmul_t: ldy = %lld is smaller than n = %lld", (long long)ldy, (long long)n);
  if (m == 0 || n == 0) return XNQ_OK;
  if (!image || !y) return fail(XNQ_ERR_NULL, "matmul_t: image or y is NULL");
  if (!aligned(image, 256)) return fail(XNQ_ERR_ALIGN, "matmul_t: the activation image must be 256-byte aligned");
  if (!aligned(y, type_size(y_dtype))) return fail(XNQ_ERR_ALIGN, "matmul_t: y is not aligned to its element size");
  const int adt = act_dtype_for(w->v.dtype);
  int rc;
  // two rows and up: the integer tensor-core kernel, where the caller gave it its scratch (it re-lays the image out)
  if (use_imma(w, m) && workspace && aligned(workspace, 256) && ws_bytes >= imma_workspace_bytes(m, k, n))
    return launch_imma(w->v, image, XNQ_ACT_IMAGE, m, k, y, y_dtype, ldy, workspace, s);
  if (matvec_tma_enabled() && matvec_tma_supported(w->v, m)) {
    profile_mark(s, true);
    rc = launch_matvec_tma(w->v, image, XNQ_ACT_IMAGE, y, y_dtype, s);
    profile_mark(s, false);
    return rc;
  }
  bool use_mma = false;
  const int64_t pass = small_batch_pass(w, m, y_dtype, &use_mma);
  if (pass == 0) return fail(XNQ_ERR_SIZE, "matmul_t: k = %lld is too large for the shared-memory staging of one activation row", (long long)k);
  const ActView all = act_view(const_cast<void *>(image), m, k, adt);
  const int blk = adt == XNQ_Q8_0 ? QK : QK_K;
  const size_t yes = type_size(y_dtype);
  for (int64_t r0 = 0; r0 < m; r0 += pass) {
    ActView a = all;
    a.m = (m - r0) < pass ? (m - r0) : pass;
    a.q += r0 * k;
    a.d += r0 * (k / blk);
    a.bsum += r0 * (k / 16);
    profile_mark(s, true);
    rc = use_mma ? launch_matvec_mma(w->v, a, static_cast<char *>(y) + (size_t)r0 * ldy * yes, y_dtype, ldy, s)
                 : launch_matvec(w->v, a, static_cast<char *>(y) + (size_t)r0 * ldy * yes, y_dtype, ldy, s);
    profile_mark(s, false);
    if (rc != XNQ_OK) return rc;
  }
  return XNQ_OK;
}

extern "C" {

const char *xnq_last_error(void) { return g_err; }
int xnq_version(void) { return XNQ_VERSION; }
int xnq_type_size(int dt) { return (is_weight_dtype(dt) || dt == XNQ_Q8K || dt == XNQ_Q8_1 || is_float_dtype(dt)) ? type_size(dt) : -1; }
int xnq_block_size(int dt) { return (is_weight_dtype(dt) || dt == XNQ_Q8K || dt == XNQ_Q8_1 || is_float_dtype(dt)) ? block_size(dt) : -1; }

uint64_t xnq_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int xnq_profile_begin(int max_launches) {
  clear_error();
  if (max_launches <= 0 || max_launches > (1 << 20)) return fail(XNQ_ERR_SIZE, "profile_begin: max_launches = %d", max_launches);
  Profile &p = g_prof;
  for (cudaEvent_t e : p.ev) cudaEventDestroy(e);
  p.ev.clear();
  p.used = 0;
  p.ev.resize((size_t)max_launches * 2);
  for (auto &e : p.ev) XNQ_CUDA(cudaEventCreate(&e));
  p.on = true;
  return XNQ_OK;
}

int xnq_profile_end(double *total_ms, int *launches) {
  clear_error();
  Profile &p = g_prof;
  if (!p.on) return fail(XNQ_ERR_SHAPE, "profile_end without profile_begin");
  p.on = false;
  double total = 0.0;
  int rc = XNQ_OK;
  for (size_t i = 0; i + 1 < p.used; i += 2) {
    float ms = 0.f;
    cudaError_t e = cudaEventSynchronize(p.ev[i + 1]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, p.ev[i], p.ev[i + 1]);
    if (e != cudaSuccess) {
      rc = fail(XNQ_ERR_CUDA, "profile_end: %s", cudaGetErrorString(e));
      break;
    }
    total += ms;
  }
  if (total_ms) *total_ms = total;
  if (launches) *launches = (int)(p.used / 2);
  for (cudaEvent_t e : p.ev) cudaEventDestroy(e);
  p.ev.clear();
  p.used = 0;
  return rc;
}

int xnq_init(int device) {
  clear_error();
  int count = 0;
  XNQ_CUDA(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count) return fail(XNQ_ERR_SHAPE, "xnq_init: device %d out of range (%d visible)", device, count);
  cudaDeviceProp prop;
  XNQ_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(XNQ_ERR_UNSUPPORTED, "xnq_init: device %d is sm_%d%d; this library is built for sm_100a only and has no fallback",
                device, prop.major, prop.minor);
  XNQ_CUDA(cudaSetDevice(device));
  int rc;
  if ((rc = layout_init(device)) != XNQ_OK) return rc;
  if ((rc = quantize_init(device)) != XNQ_OK) return rc;
  if ((rc = matvec_init(device)) != XNQ_OK) return rc;
  if ((rc = matvec_mma_init(device)) != XNQ_OK) return rc;
  if ((rc = matvec_tma_init(device)) != XNQ_OK) return rc;
  if ((rc = prefill_init(device)) != XNQ_OK) return rc;
  if ((rc = imma_init(device)) != XNQ_OK) return rc;
  if ((rc = decoder_ops_init()) != XNQ_OK) return rc;
  if ((rc = generic_init(device)) != XNQ_OK) return rc;
  return XNQ_OK;
}

int xnq_device_status(unsigned int *bits) {
  clear_error();
  if (!bits) return fail(XNQ_ERR_NULL, "device_status: bits is NULL");
  unsigned int mv = 0, pf = 0, im = 0, dc = 0;
  int rc = matvec_status(&mv);
  if (rc == XNQ_OK) rc = prefill_status(&pf);
  if (rc == XNQ_OK) rc = imma_status(&im);
  if (rc == XNQ_OK) rc = decoder_status(&dc);
  *bits = (mv & 0xffu) | ((pf & 0xffu) << 8) | ((im & 0xffu) << 16) | ((dc & 0xffu) << 24);
  return rc;
}

int xnq_device_check_record(unsigned long long out[8]) {
  clear_error();
  if (!out) return fail(XNQ_ERR_NULL, "device_check_record: out is NULL");
  return matvec_check_record(out);
}

int xnq_set_option(const char *name, int value) {
  clear_error();
  if (!name) return fail(XNQ_ERR_NULL, "set_option: name is NULL");
  if (std::strcmp(name, "matvec_tma") == 0) {
    g_opt_matvec_tma.store(value != 0);
    return XNQ_OK;
  }
  if (std::strcmp(name, "imma_fold") == 0) {
    imma_set_fold(value);
    return XNQ_OK;
  }
  if (std::strcmp(name, "imma") == 0) {
    g_opt_imma.store(value);
    return XNQ_OK;
  }
  if (std::strcmp(name, "matvec_mma") == 0) {
    g_opt_matvec_mma.store(value);
    return XNQ_OK;
  }
  if (std::strcmp(name, "host_direct_y") == 0) {
    g_opt_host_direct_y.store(value);
    return XNQ_OK;
  }
  if (std::strcmp(name, "gather_cta_fence") == 0) {
    g_opt_gather_cta_fence.store(value);
    return XNQ_OK;
  }
  return fail(XNQ_ERR_UNSUPPORTED, "set_option: unknown option '%s'", name);
}

int xnq_weight_upload_rows(int dtype, const void *blocks, size_t nbytes, int64_t n_total, int64_t k, int64_t row0, int64_t n_rows,
                           void *stream, xnq_weight **out) {
  clear_error();
  if (!out) return fail(XNQ_ERR_NULL, "weight_upload: out is NULL");
  *out = nullptr;
  if (!is_weight_dtype(dtype)) return fail(XNQ_ERR_DTYPE, "weight_upload: ggml dtype %d is not a quantized weight format (Q4_0 2, Q4_1 3, Q5_0 6, Q5_1 7, Q8_0 8, Q2K 10, Q3K 11, Q4K 12, Q5K 13, Q6K 14)", dtype);
  if (n_total < 0 || k <= 0 || row0 < 0 || n_rows < 0 || row0 + n_rows > n_total)
    return fail(XNQ_ERR_SHAPE, "weight_upload: bad shape n_total=%lld k=%lld rows [%lld, +%lld)", (long long)n_total, (long long)k,
                (long long)row0, (long long)n_rows);
  const int bs = block_size(dtype);
  if (k % bs != 0) return fail(XNQ_ERR_SHAPE, "weight_upload: k = %lld is not a multiple of the %d-value block", (long long)k, bs);
  if (n_total > INT32_MAX || k > INT32_MAX) return fail(XNQ_ERR_SHAPE, "weight_upload: n or k exceeds 2^31-1");
  const size_t want = (size_t)n_rows * (k / bs) * type_size(dtype);
  if (nbytes != want)
    return fail(XNQ_ERR_SIZE, "weight_upload: [%lld, %lld] wants %zu bytes of blocks, got %zu", (long long)n_rows, (long long)k, want, nbytes);
  if (!blocks && nbytes) return fail(XNQ_ERR_NULL, "weight_upload: blocks is NULL");

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  xnq_weight *w = new (std::nothrow) xnq_weight();
  if (!w) return fail(XNQ_ERR_SIZE, "weight_upload: out of host memory");
  std::memset(w, 0, sizeof(*w));
  XNQ_CUDA(cudaGetDevice(&w->device));
  w->n_total = n_total;
  w->row0 = row0;
  w->wscale = 1.0f;
  if (is_generic_dtype(dtype)) { // held exactly as in the file: canonical blocks, row after row
    const size_t alloc = nbytes ? ((nbytes + 255) & ~(size_t)255) : 256;
    cudaError_t ge = cudaMalloc(&w->base, alloc);
    if (ge == cudaSuccess && nbytes) ge = cudaMemcpyAsync(w->base, blocks, nbytes, cudaMemcpyDefault, s);
    if (ge == cudaSuccess) ge = cudaStreamSynchronize(s);
    if (ge != cudaSuccess) {
      if (w->base) cudaFree(w->base);
      delete w;
      return fail(XNQ_ERR_CUDA, "weight_upload: %s", cudaGetErrorString(ge));
    }
    w->bytes = alloc;
    w->v.dtype = dtype, w->v.n = n_rows, w->v.k = k, w->v.dstride = 0;
    w->v.qs = static_cast<const uint8_t *>(w->base);
    *out = w;
    return XNQ_OK;
  }
  const Plan p = plan_for(dtype, n_rows, k);
  cudaError_t e = cudaMalloc(&w->base, p.total);
  if (e != cudaSuccess) {
    delete w;
    return fail(XNQ_ERR_CUDA, "weight_upload: cudaMalloc(%zu) failed: %s", p.total, cudaGetErrorString(e));
  }
  w->bytes = p.total;
  char *b = static_cast<char *>(w->base);
  w->v.dtype = dtype;
  w->v.n = n_rows;
  w->v.k = k;
  w->v.dstride = p.dstride;
  w->v.qs = reinterpret_cast<const uint8_t *>(b + p.qs);
  w->v.qh = dtype == XNQ_Q6K ? reinterpret_cast<const uint8_t *>(b + p.qh) : nullptr;
  w->v.sc = dtype == XNQ_Q6K ? reinterpret_cast<const int8_t *>(b + p.sc) : nullptr;
  w->v.d = dtype == XNQ_Q4K ? nullptr : reinterpret_cast<const __half *>(b + p.d);

  int rc = XNQ_OK;
  void *staging = nullptr;
  do {
    if ((e = cudaMemsetAsync(w->base, 0, p.total, s)) != cudaSuccess) break;
    if (nbytes == 0) break;
    if ((e = cudaMalloc(&staging, nbytes)) != cudaSuccess) break;
    if ((e = cudaMemcpyAsync(staging, blocks, nbytes, cudaMemcpyDefault, s)) != cudaSuccess) break;
    rc = launch_relayout(w->v, static_cast<const uint8_t *>(staging), s);
    if (rc != XNQ_OK) break;
    // largest |weight| -> the power-of-two scale of the fp16 prefill path (the staging buffer's first word is free now)
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) break;
    rc = launch_max_abs(w->v, static_cast<float *>(staging), s);
    if (rc != XNQ_OK) break;
    float maxabs = 0.f;
    if ((e = cudaMemcpyAsync(&maxabs, staging, sizeof(float), cudaMemcpyDeviceToHost, s)) != cudaSuccess) break;
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) break;
    if (maxabs > 0.f) {
      int ex = 0;
      (void)std::frexp(maxabs, &ex); // maxabs = f * 2^ex, f in [0.5, 1)
      w->wscale = std::ldexp(1.0f, 10 - ex);
    }
  } while (0);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (staging) cudaFree(staging);
  if (e != cudaSuccess || rc != XNQ_OK) {
    cudaFree(w->base);
    delete w;
    if (rc != XNQ_OK) return rc;
    return fail(XNQ_ERR_CUDA, "weight_upload: %s", cudaGetErrorString(e));
  }
  *out = w;
  return XNQ_OK;
}

int xnq_weight_upload(int dtype, const void *blocks, size_t nbytes, int64_t n, int64_t k, int shard_rank, int shard_count, void *stream,
                      xnq_weight **out) {
  clear_error();
  if (out) *out = nullptr;
  if (!is_weight_dtype(dtype)) return fail(XNQ_ERR_DTYPE, "weight_upload: ggml dtype %d is not a quantized weight format (Q4_0 2, Q4_1 3, Q5_0 6, Q5_1 7, Q8_0 8, Q2K 10, Q3K 11, Q4K 12, Q5K 13, Q6K 14)", dtype);
  if (shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count)
    return fail(XNQ_ERR_SHAPE, "weight_upload: shard %d of %d", shard_rank, shard_count);
  if (n < 0 || k <= 0 || k % block_size(dtype) != 0)
    return fail(XNQ_ERR_SHAPE, "weight_upload: bad shape [%lld, %lld] for a %d-value block", (long long)n, (long long)k, block_size(dtype));
  if (n % shard_count != 0) return fail(XNQ_ERR_SHAPE, "weight_upload: n = %lld does not divide over %d shards", (long long)n, shard_count);
  const size_t row_bytes = (size_t)(k / block_size(dtype)) * type_size(dtype);
  if (nbytes != (size_t)n * row_bytes)
    return fail(XNQ_ERR_SIZE, "weight_upload: [%lld, %lld] wants %zu bytes of blocks, got %zu", (long long)n, (long long)k, (size_t)n * row_bytes,
                nbytes);
  if (!blocks && nbytes) return fail(XNQ_ERR_NULL, "weight_upload: blocks is NULL");
  const int64_t rows = n / shard_count, row0 = rows * shard_rank;
  return xnq_weight_upload_rows(dtype, static_cast<const char *>(blocks) + (size_t)row0 * row_bytes, (size_t)rows * row_bytes, n, k, row0, rows,
                                stream, out);
}

int xnq_weight_free(xnq_weight *w) {
  clear_error();
  if (!w) return XNQ_OK;
  if (w->base) cudaFree(w->base);
  if (w->stage_dev) cudaFree(w->stage_dev);
  if (w->stage_host) cudaFreeHost(w->stage_host);
  delete w;
  return XNQ_OK;
}

int xnq_weight_info(const xnq_weight *w, int *dtype, int64_t *n_total, int64_t *n_local, int64_t *row0, int64_t *k, size_t *device_bytes) {
  clear_error();
  if (!w) return fail(XNQ_ERR_NULL, "weight_info: weight is NULL");
  if (dtype) *dtype = w->v.dtype;
  if (n_total) *n_total = w->n_total;
  if (n_local) *n_local = w->v.n;
  if (row0) *row0 = w->row0;
  if (k) *k = w->v.k;
  if (device_bytes) *device_bytes = w->bytes;
  return XNQ_OK;
}

int xnq_weight_dequantize(const xnq_weight *w, int out_dtype, void *dst, void *stream) {
  clear_error();
  if (!w) return fail(XNQ_ERR_NULL, "dequantize: weight is NULL");
  if (!is_float_dtype(out_dtype)) return fail(XNQ_ERR_DTYPE, "dequantize: output dtype %d is not f32/f16/bf16", out_dtype);
  if (w->v.n == 0) return XNQ_OK;
  if (!dst) return fail(XNQ_ERR_NULL, "dequantize: dst is NULL");
  if (is_generic_dtype(w->v.dtype)) return launch_generic_dequantize(w->v, out_dtype, dst, static_cast<cudaStream_t>(stream));
  return launch_dequantize(w->v, out_dtype, dst, static_cast<cudaStream_t>(stream));
}

int xnq_weight_canonical_bytes(const xnq_weight *w, void *host_dst, size_t nbytes, void *stream) {
  clear_error();
  if (!w) return fail(XNQ_ERR_NULL, "canonical_bytes: weight is NULL");
  const size_t want = (size_t)w->v.n * (w->v.k / block_size(w->v.dtype)) * type_size(w->v.dtype);
  if (nbytes != want) return fail(XNQ_ERR_SIZE, "canonical_bytes: the held rows are %zu bytes, buffer is %zu", want, nbytes);
  if (want == 0) return XNQ_OK;
  if (!host_dst) return fail(XNQ_ERR_NULL, "canonical_bytes: host_dst is NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_generic_dtype(w->v.dtype)) { // already canonical on the device
    XNQ_CUDA(cudaMemcpyAsync(host_dst, w->v.qs, want, cudaMemcpyDeviceToHost, s));
    XNQ_CUDA(cudaStreamSynchronize(s));
    return XNQ_OK;
  }
  void *staging = nullptr;
  XNQ_CUDA(cudaMalloc(&staging, want));
  int rc = launch_to_canonical(w->v, static_cast<uint8_t *>(staging), s);
  cudaError_t e = cudaSuccess;
  if (rc == XNQ_OK) e = cudaMemcpyAsync(host_dst, staging, want, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(staging);
  if (rc != XNQ_OK) return rc;
  if (e != cudaSuccess) return fail(XNQ_ERR_CUDA, "canonical_bytes: %s", cudaGetErrorString(e));
  return XNQ_OK;
}

int xnq_quantize_act(int act_dtype, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx, void *dst, void *stream) {
  clear_error();
  if (act_dtype != XNQ_Q8_0 && act_dtype != XNQ_Q8_1 && act_dtype != XNQ_Q8K)
    return fail(XNQ_ERR_DTYPE, "quantize_act: %d is not an activation block format (Q8_0=8, Q8_1=9, Q8K=15)", act_dtype);
  const int bs = block_size(act_dtype);
  if (k <= 0 || k % bs != 0) return fail(XNQ_ERR_SHAPE, "quantize_act: k = %lld is not a multiple of the %d-value block", (long long)k, bs);
  int rc = check_activations("quantize_act", x, x_dtype, m, k, ldx);
  if (rc != XNQ_OK) return rc;
  if (m == 0) return XNQ_OK;
  if (!dst) return fail(XNQ_ERR_NULL, "quantize_act: dst_blocks is NULL");
  if (!aligned(dst, 4)) return fail(XNQ_ERR_ALIGN, "quantize_act: dst_blocks must be 4-byte aligned");
  if (act_dtype == XNQ_Q8_1) return launch_quantize_q8_1(x, x_dtype, m, k, ldx, dst, static_cast<cudaStream_t>(stream));
  return launch_quantize_act_blocks(act_dtype, x, x_dtype, m, k, ldx, dst, static_cast<cudaStream_t>(stream));
}

size_t xnq_act_operand_bytes(int64_t m, int64_t k) {
  if (m <= 0 || m > IMMA_MAX_M || k <= 0 || k % 256) return 0;
  return operand_image_bytes(m, k);
}

size_t xnq_act_image_bytes(int act_dtype, int64_t m, int64_t k) {
  if ((act_dtype != XNQ_Q8_0 && act_dtype != XNQ_Q8K) || m <= 0 || k <= 0) return 0;
  return act_workspace_bytes(m, k, act_dtype);
}

int xnq_quantize_act_image(int act_dtype, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx, void *image, void *stream) {
  clear_error();
  if (act_dtype != XNQ_Q8_0 && act_dtype != XNQ_Q8K)
    return fail(XNQ_ERR_DTYPE, "quantize_act_image: %d is not an activation block format (Q8_0=8, Q8K=15)", act_dtype);
  const int bs = block_size(act_dtype);
  if (k <= 0 || k % bs != 0) return fail(XNQ_ERR_SHAPE, "quantize_act_image: k = %lld is not a multiple of the %d-value block", (long long)k, bs);
  int rc = check_activations("quantize_act_image", x, x_dtype, m, k, ldx);
  if (rc != XNQ_OK) return rc;
  if (m == 0) return XNQ_OK;
  if (!image) return fail(XNQ_ERR_NULL, "quantize_act_image: image is NULL");
  if (!aligned(image, 256)) return fail(XNQ_ERR_ALIGN, "quantize_act_image: image must be 256-byte aligned");
  return launch_quantize_act_planar(act_view(image, m, k, act_dtype), x, x_dtype, ldx, static_cast<cudaStream_t>(stream));
}

int xnq_quantize_weight(int ggml_dtype, const float *x_dev, int64_t n, int64_t k, void *blocks_dev, void *stream) {
  clear_error();
  if (!is_fast_dtype(ggml_dtype)) return fail(XNQ_ERR_DTYPE, "quantize_weight: dtype %d is not Q4_0/Q8_0/Q4K/Q6K (the other formats have no device quantizer)", ggml_dtype);
  const int bs = block_size(ggml_dtype);
  if (n < 0 || k <= 0 || k % bs != 0)
    return fail(XNQ_ERR_SHAPE, "quantize_weight: quantized tensor must have their last dim divisible by block size [%lld, %lld] %d", (long long)n, (long long)k, bs);
  if (n == 0) return XNQ_OK;
  if (!x_dev || !blocks_dev) return fail(XNQ_ERR_NULL, "quantize_weight: x_dev or blocks_dev is NULL");
  if (!aligned(x_dev, 16) || !aligned(blocks_dev, 16)) return fail(XNQ_ERR_ALIGN, "quantize_weight: x_dev and blocks_dev must be 16-byte aligned");
  return launch_quantize_weight(ggml_dtype, x_dev, n, k, blocks_dev, static_cast<cudaStream_t>(stream));
}

int xnq_hint_next_weight(const xnq_weight *w) {
  clear_error();
  matvec_hint_next(w);
  return XNQ_OK;
}

int xnq_matvec_normed(const xnq_weight *w, const float *x_in, const float *delta, int delta_parts, const float *norm_weight, float eps, float *x_out, void *y,
                      int y_dtype, const xnq_comm *await, void *stream) {
  clear_error();
  if (!w || !x_in || !norm_weight || !x_out || !y) return fail(XNQ_ERR_NULL, "matvec_normed: NULL argument");
  if (x_in == x_out) return fail(XNQ_ERR_SHAPE, "matvec_normed: x_out must not be x_in (every CTA reads x_in while one writes x_out)");
  if ((delta && delta_parts < 1) || (!delta && delta_parts != 0)) return fail(XNQ_ERR_SHAPE, "matvec_normed: delta_parts = %d", delta_parts);
  if (!is_float_dtype(y_dtype)) return fail(XNQ_ERR_DTYPE, "matvec_normed: output dtype %d is not f32/f16/bf16", y_dtype);
  if (((uintptr_t)x_in | (uintptr_t)delta | (uintptr_t)norm_weight | (uintptr_t)x_out) & 15) return fail(XNQ_ERR_ALIGN, "matvec_normed: pointers must be 16-byte aligned");
  if (!aligned(y, type_size(y_dtype))) return fail(XNQ_ERR_ALIGN, "matvec_normed: y is not aligned to its element size");
  if (w->v.k % 8 || !matvec_tma_supported(w->v, 1) || matvec_tma_wants_image(w->v))
    return fail(XNQ_ERR_UNSUPPORTED, "matvec_normed: rows of %lld values (the fused prologue serves rows of up to 4096 values; use xnq_add_rmsnorm + xnq_matmul_t)", (long long)w->v.k);
  if (w->v.n == 0) return XNQ_OK;
  NormArgs na;
  na.x_in = x_in, na.delta = delta, na.parts = delta ? delta_parts : 0, na.weight = norm_weight, na.eps = eps, na.x_out = x_out;
  if (await) {
    const int wrc = comm_fill_wait(await, &na);
    if (wrc != XNQ_OK) return wrc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  profile_mark(s, true);
  const int rc = launch_matvec_tma(w->v, x_in, XNQ_F32, y, y_dtype, s, nullptr, &na);
  profile_mark(s, false);
  return rc;
}

size_t xnq_matmul_workspace_bytes(const xnq_weight *w, int64_t max_m) {
  if (!w || max_m <= 0) return 0;
  if (is_generic_dtype(w->v.dtype)) return generic_workspace_bytes(w->v, max_m);
  const int64_t rows = max_m < MATVEC_MAX_M ? max_m : MATVEC_MAX_M;
  size_t decode = act_workspace_bytes(rows, w->v.k, act_dtype_for(w->v.dtype));
  if (max_m >= 2 && imma_supported(w->v, 2)) decode = std::max(decode, imma_workspace_bytes(std::min<int64_t>(max_m, IMMA_MAX_M), w->v.k, w->v.n));
  if (max_m <= MATVEC_MAX_M) return decode;
  const size_t prefill = prefill_workspace_bytes(max_m, w->v.k, w->v.n); // m > 16 runs on the tensor cores
  return prefill > decode ? prefill : decode;
}

int xnq_matmul_t(const xnq_weight *w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy, void *workspace,
                 size_t ws_bytes, void *stream) {
  clear_error();
  if (!w) return fail(XNQ_ERR_NULL, "matmul_t: weight is NULL");
  const int64_t k = w->v.k, n = w->v.n;
  if (x_dtype == XNQ_ACT_IMAGE && is_generic_dtype(w->v.dtype)) return fail(XNQ_ERR_UNSUPPORTED, "matmul_t: dtype %d takes float activations only (no activation image)", w->v.dtype);
  if (x_dtype == XNQ_ACT_OPERAND) return matmul_from_operand(w, x, m, y, y_dtype, ldy, workspace, ws_bytes, static_cast<cudaStream_t>(stream));
  if (x_dtype == XNQ_ACT_IMAGE) return matmul_from_image(w, x, m, y, y_dtype, ldy, workspace, ws_bytes, static_cast<cudaStream_t>(stream));
  int rc = check_activations("matmul_t", x, x_dtype, m, k, ldx);
  if (rc != XNQ_OK) return rc;
  if (!is_float_dtype(y_dtype)) return fail(XNQ_ERR_DTYPE, "matmul_t: output dtype %d is not f32/f16/bf16", y_dtype);
  if (ldy < n) return fail(XNQ_ERR_SHAPE, "matmul_t: ldy = %lld is smaller than n = %lld", (long long)ldy, (long long)n);
  if (m == 0 || n == 0) return XNQ_OK;
  if (!y) return fail(XNQ_ERR_NULL, "matmul_t: y is NULL");
  if (!aligned(y, type_size(y_dtype))) return fail(XNQ_ERR_ALIGN, "matmul_t: y is not aligned to its element size");
  const size_t need = xnq_matmul_workspace_bytes(w, m);
  if (!workspace) return fail(XNQ_ERR_NULL, "matmul_t: workspace is NULL (need %zu bytes)", need);
  if (!aligned(workspace, 256)) return fail(XNQ_ERR_ALIGN, "matmul_t: workspace must be 256-byte aligned");
  if (ws_bytes < need) return fail(XNQ_ERR_SIZE, "matmul_t: workspace has %zu bytes, m = %lld needs %zu", ws_bytes, (long long)m, need);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_generic_dtype(w->v.dtype)) return launch_generic_matmul(w->v, x, x_dtype, m, ldx, y, y_dtype, ldy, workspace, s);
  if (g_opt_matvec_tma.load(std::memory_order_relaxed) && matvec_tma_supported(w->v, m)) {
    // decode fast path: one kernel; activations quantized in its prologue (k <= 4096, no scratch) or, for longer
    // rows, by the stand-alone quantizer into the workspace as an activation image
    const void *xin = x;
    int xin_dtype = x_dtype;
    if (matvec_tma_wants_image(w->v)) {
      const ActView a = act_view(workspace, 1, k, act_dtype_for(w->v.dtype));
      if ((rc = launch_quantize_act_planar(a, x, x_dtype, ldx, s)) != XNQ_OK) return rc;
      xin = workspace;
      xin_dtype = XNQ_ACT_IMAGE;
    }
    profile_mark(s, true);
    rc = launch_matvec_tma(w->v, xin, xin_dtype, y, y_dtype, s);
    profile_mark(s, false);
    return rc;
  }
  if (use_imma(w, m)) return launch_imma(w->v, x, x_dtype, m, ldx, y, y_dtype, ldy, workspace, s); // exact integer dots on the tensor cores
  if (m > MATVEC_MAX_M) return launch_prefill(w->v, w->wscale, x, x_dtype, m, ldx, y, y_dtype, ldy, workspace, s);
  bool use_mma = false;
  const int64_t pass = small_batch_pass(w, m, y_dtype, &use_mma);
  if (pass == 0) return fail(XNQ_ERR_SIZE, "matmul_t: k = %lld is too large for the shared-memory staging of one activation row", (long long)k);
  const int adt = act_dtype_for(w->v.dtype);
  const size_t xes = type_size(x_dtype), yes = type_size(y_dtype);
  for (int64_t r0 = 0; r0 < m; r0 += pass) {
    const int64_t rows = (m - r0) < pass ? (m - r0) : pass;
    ActView a = act_view(workspace, rows, k, adt);
    const char *xp = static_cast<const char *>(x) + (size_t)r0 * ldx * xes;
    char *yp = static_cast<char *>(y) + (size_t)r0 * ldy * yes;
    if ((rc = launch_quantize_act_planar(a, xp, x_dtype, ldx, s)) != XNQ_OK) return rc;
    profile_mark(s, true);
    rc = use_mma ? launch_matvec_mma(w->v, a, yp, y_dtype, ldy, s) : launch_matvec(w->v, a, yp, y_dtype, ldy, s);
    profile_mark(s, false);
    if (rc != XNQ_OK) return rc;
  }
  return XNQ_OK;
}

// device staging of xnq_linear_forward_host for up to m rows: activations | result | bias | matmul workspace
static size_t host_staging_bytes(const xnq_weight *w, int64_t m, size_t *xb, size_t *yb, size_t *bb, size_t *wsb) {
  const int64_t k = w->v.k, n = w->v.n;
  *xb = up256((size_t)m * k * 4), *yb = up256((size_t)m * n * 4), *bb = up256((size_t)n * 4);
  *wsb = up256(xnq_matmul_workspace_bytes(w, m));
  return *xb + *yb + *bb + *wsb;
}

int xnq_weight_reserve_host_staging(xnq_weight *w, int64_t max_m) {
  clear_error();
  if (!w) return fail(XNQ_ERR_NULL, "reserve_host_staging: weight is NULL");
  if (max_m < 1) return fail(XNQ_ERR_SHAPE, "reserve_host_staging: max_m = %lld", (long long)max_m);
  size_t xb, yb, bb, wsb;
  const size_t need = host_staging_bytes(w, max_m, &xb, &yb, &bb, &wsb);
  if (w->stage_dev_bytes >= need) return XNQ_OK;
  if (w->stage_dev) cudaFree(w->stage_dev);
  w->stage_dev = nullptr;
  w->stage_dev_bytes = 0;
  XNQ_CUDA(cudaMalloc(&w->stage_dev, need));
  w->stage_dev_bytes = need;
  return XNQ_OK;
}

int xnq_linear_forward_host(xnq_weight *w, const float *x_host, int64_t m, const float *bias_host, float *y_host, void *stream) {
  clear_error();
  if (!w) return fail(XNQ_ERR_NULL, "linear_forward_host: weight is NULL");
  if (m < 0) return fail(XNQ_ERR_SHAPE, "linear_forward_host: m = %lld", (long long)m);
  const int64_t k = w->v.k, n = w->v.n;
  if (m == 0 || n == 0) return XNQ_OK;
  if (!x_host || !y_host) return fail(XNQ_ERR_NULL, "linear_forward_host: x_host or y_host is NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  size_t xb, yb, bb, wsb;
  const size_t need = host_staging_bytes(w, m, &xb, &yb, &bb, &wsb);
  if (w->stage_dev_bytes < need) { // not reserved ahead of time: grow now (this allocates, so it must not happen inside a stream capture)
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
      return fail(XNQ_ERR_UNSUPPORTED, "linear_forward_host: m = %lld needs %zu bytes of staging, %zu are reserved, and the stream is being captured; "
                  "call xnq_weight_reserve_host_staging first", (long long)m, need, w->stage_dev_bytes);
    const int rc0 = xnq_weight_reserve_host_staging(w, m);
    if (rc0 != XNQ_OK) return rc0;
  }
  char *base = static_cast<char *>(w->stage_dev);
  float *xd = reinterpret_cast<float *>(base);
  float *yd = reinterpret_cast<float *>(base + xb);
  float *bd = reinterpret_cast<float *>(base + xb + yb);
  void *ws = base + xb + yb + bb;
  XNQ_CUDA(cudaMemcpyAsync(xd, x_host, (size_t)m * k * 4, cudaMemcpyHostToDevice, s));
  if (bias_host) XNQ_CUDA(cudaMemcpyAsync(bd, bias_host, (size_t)n * 4, cudaMemcpyHostToDevice, s));
  // A page-locked result buffer is written by the kernel itself (posted stores over the host link), which
  // saves the device-to-host copy and its launch; anything else goes through the staging buffer. The
  // activations are always copied in: every CTA reads all of x, which must not cross the host link 148 times.
  float *y_direct = nullptr;
  // (not where the small-batch kernel splits k between CTAs that add into y atomically: that needs device memory)
  if (!bias_host && m <= MATVEC_MAX_M && !(m >= 5 && matvec_mma_accumulates_in_y(w->v, m)) && g_opt_host_direct_y.load(std::memory_order_relaxed)) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, y_host) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer &&
        (reinterpret_cast<uintptr_t>(attr.devicePointer) & 15) == 0)
      y_direct = static_cast<float *>(attr.devicePointer);
    else
      (void)cudaGetLastError(); // an unregistered pointer is not an error here
  }
  int rc = xnq_matmul_t(w, xd, XNQ_F32, m, k, y_direct ? y_direct : yd, XNQ_F32, n, ws, wsb, s);
  if (rc != XNQ_OK) return rc;
  if (bias_host && (rc = launch_add_bias(yd, bd, m, n, n, s)) != XNQ_OK) return rc;
  if (!y_direct) XNQ_CUDA(cudaMemcpyAsync(y_host, yd, (size_t)m * n * 4, cudaMemcpyDeviceToHost, s));
  XNQ_CUDA(cudaStreamSynchronize(s));
  return XNQ_OK;
}

} // extern "C"
