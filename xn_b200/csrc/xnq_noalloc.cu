// xnq_matmul_t_static: the small-batch quantized matmul for callers that must not allocate.
//
// Who this is for. Some hosts of this library cannot hand it a scratch buffer and cannot let it call
// cudaMalloc either: a serving loop that has promised its device memory to its own pool (xn's CUDA
// backend gives every byte to cudarc's stream-ordered allocator), a decode step that is being
// recorded into a CUDA graph (an allocation there is refused or, worse, silently serializes the
// device), or a plugin that runs under a fixed memory budget it may not exceed. For them the
// quantized-activation scratch that xnq_matmul_t takes from the caller lives here instead, in one
// fixed array inside the library's own device image.
//
// The array is a file-scope __device__ object: every GPU that loads the library carries its
// SCRATCH_BYTES (128 KiB) from load until the process exits, whether or not this entry is used.
// In host code the array's name is only a stand-in for the symbol, not a device address, so the
// address is looked up once per device with cudaGetSymbolAddress (that device being current) and
// that pointer is what the kernels receive.
#include <mutex>

#include "xnq_common.cuh"

namespace xnq {
namespace {

constexpr size_t SCRATCH_BYTES = 128 * 1024; // quantized activations (1.25 bytes per element) of the rows of one pass
static __device__ __align__(256) unsigned char g_static_scratch[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_setup_mutex;
void *g_scratch_ptr[MAX_DEVICES] = {nullptr}; // device address of g_static_scratch, per device

// First use on a device: resolve the array's device address (no allocation; the array already exists).
int scratch_for_device(int device, void **out) {
  if (device < 0 || device >= MAX_DEVICES) return fail(XNQ_ERR_UNSUPPORTED, "matmul_t_static: device %d is beyond the %d this entry tracks", device, MAX_DEVICES);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[device]) {
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch); // for the CURRENT device, which the caller checked is `device`
    if (e != cudaSuccess || !p) return fail(XNQ_ERR_CUDA, "matmul_t_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_ptr[device] = p;
  }
  *out = g_scratch_ptr[device];
  return XNQ_OK;
}

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

} // namespace
} // namespace xnq

using namespace xnq;

extern "C" int xnq_matmul_t_static(const xnq_weight *w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y, int y_dtype, int64_t ldy,
                                   void *stream) {
  clear_error();
  if (!w) return fail(XNQ_ERR_NULL, "matmul_t_static: weight is NULL");
  const int64_t k = w->v.k, n = w->v.n;
  if (!is_fast_dtype(w->v.dtype)) return fail(XNQ_ERR_UNSUPPORTED, "matmul_t_static: weight dtype %d is served by xnq_matmul_t only", w->v.dtype);
  if (!is_float_dtype(x_dtype) || !is_float_dtype(y_dtype)) return fail(XNQ_ERR_DTYPE, "matmul_t_static: x / y dtype must be f32, f16 or bf16");
  if (m < 0 || m > MATVEC_MAX_M)
    return fail(XNQ_ERR_SIZE, "matmul_t_static: m = %lld; this entry serves 0..%d rows (larger batches need xnq_matmul_t and a caller-owned workspace)",
                (long long)m, MATVEC_MAX_M);
  if (ldx < k || ldy < n) return fail(XNQ_ERR_SHAPE, "matmul_t_static: ldx = %lld / ldy = %lld are smaller than k = %lld / n = %lld", (long long)ldx,
                                      (long long)ldy, (long long)k, (long long)n);
  if (m == 0 || n == 0) return XNQ_OK;
  if (!x || !y) return fail(XNQ_ERR_NULL, "matmul_t_static: x or y is NULL");
  const size_t xes = type_size(x_dtype), yes = type_size(y_dtype);
  if (!aligned_to(x, 16) || (m > 1 && (ldx * xes) % 16 != 0)) return fail(XNQ_ERR_ALIGN, "matmul_t_static: activation rows must start 16-byte aligned");
  if (!aligned_to(y, yes)) return fail(XNQ_ERR_ALIGN, "matmul_t_static: y is not aligned to its element size");
  const int adt = act_dtype_for(w->v.dtype);
  bool use_mma = false;
  const int64_t pass = small_batch_pass(w, m, y_dtype, &use_mma); // a kernel that needs nothing but the quantized activations as scratch
  if (pass == 0) return fail(XNQ_ERR_SIZE, "matmul_t_static: k = %lld is too large for the shared-memory staging of one activation row", (long long)k);
  // rows per pass: what the kernel can stage AND what the built-in array can hold
  int64_t rows_at_once = m < pass ? m : pass;
  while (rows_at_once > 1 && act_workspace_bytes(rows_at_once, k, adt) > SCRATCH_BYTES) rows_at_once--;
  const size_t need = act_workspace_bytes(rows_at_once, k, adt);
  if (need > SCRATCH_BYTES)
    return fail(XNQ_ERR_SIZE, "matmul_t_static: one activation row of k = %lld needs %zu bytes of scratch; the built-in array holds %zu (use xnq_matmul_t)",
                (long long)k, need, SCRATCH_BYTES);
  int device = -1;
  XNQ_CUDA(cudaGetDevice(&device));
  if (device != w->device) return fail(XNQ_ERR_UNSUPPORTED, "matmul_t_static: the weight lives on device %d but device %d is current", w->device, device);
  void *scratch = nullptr;
  int rc = scratch_for_device(device, &scratch);
  if (rc != XNQ_OK) return rc;

  // Nothing in the array has to start at zero: the quantizer below rewrites every byte (codes, block
  // scales, 16-sums of `rows` rows) that the matvec kernel of the same pass then reads.
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int64_t r0 = 0; r0 < m; r0 += rows_at_once) {
    const int64_t rows = (m - r0) < rows_at_once ? (m - r0) : rows_at_once;
    ActView a = act_view(scratch, rows, k, adt);
    const char *xp = static_cast<const char *>(x) + (size_t)r0 * ldx * xes;
    char *yp = static_cast<char *>(y) + (size_t)r0 * ldy * yes;
    if ((rc = launch_quantize_act_planar(a, xp, x_dtype, ldx, s)) != XNQ_OK) return rc;
    rc = use_mma ? launch_matvec_mma(w->v, a, yp, y_dtype, ldy, s) : launch_matvec(w->v, a, yp, y_dtype, ldy, s);
    if (rc != XNQ_OK) return rc;
  }
  return XNQ_OK;
}
