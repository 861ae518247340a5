// N-sharded matmul with the output gather done by the kernels themselves.
//
// The reference runs on one device (xn-core/src/cuda_backend/mod.rs:141-167) and has no collective;
// the quantized matmul shards along N without any exchange except the gather of the [m, n/G] output
// slices (every output column is an independent dot product, k_quants.rs:72-75). Here that gather is
// not a separate collective: every rank owns one device allocation ("region": a row of epoch words
// followed by `nslots` output slots), maps the regions of the other ranks through CUDA IPC, and the
// matmul kernel of rank r stores its columns into the same slot of EVERY rank through those
// mappings (NVLink stores, no loads from a peer). The last CTA of the launch then publishes rank r's
// next epoch into each peer's epoch row and waits - bounded - until every peer's epoch in the local
// row has reached the same count, so a launch that has retired has a complete gathered buffer.
//
// Epoch counters live in device memory and are advanced by the kernels, so a captured CUDA graph can
// be replayed: nothing about the protocol is baked into kernel arguments.
//
// Slot reuse. Rank r reaches the stores of its gather number e only after its gather e-1 retired,
// i.e. after every peer has LAUNCHED gather e-1, which in stream order follows everything
// that peer did with the results of gathers <= e-2. So a slot may be written again as soon as one
// other gather lies in between: callers alternate between at least two slots (checked here for
// consecutive calls; a replayed graph must also end on a different slot than it starts with).
#include <cstring>

#include "xnq_common.cuh"

struct xnq_comm {
  int device, rank, world, nslots;
  size_t slot_bytes;   // rounded up to 256
  void *region;        // local: [XNQ_MAX_RANKS epoch words, padded to 256 B][slot 0][slot 1]...
  void *peer[xnq::XNQ_MAX_RANKS]; // peer[rank] == region; the others are IPC mappings
  unsigned int *ctl;   // local, not shared: {epochs sent, unused, CTAs done, late-peer bits}
  bool connected;
  int last_slot;
  int deferred;        // 1: gathers publish and retire; xnq_comm_wait awaits the peers
};

namespace xnq {
namespace {

constexpr size_t FLAG_BYTES = 256;

// Copies this rank's [m, n] column block from `src` (row stride ld_src elements; may be the rank's own
// slot) into columns [col0, col0 + n) of the slot of every rank except `skip`, then publishes the
// epoch and waits for the peers'. Used when the producing kernel could not store remotely itself.
__global__ void __launch_bounds__(256) gather_push_kernel(GatherArgs g, const void *src_v, int64_t ld_src, int64_t m, int64_t n, int es, int skip) {
  const int64_t row_bytes = n * es;
  const char *src = static_cast<const char *>(src_v);
  const bool vec = ((g.col0 * es) % 16 == 0) && ((g.ld * es) % 16 == 0) && (row_bytes % 16 == 0) && ((ld_src * es) % 16 == 0) &&
                   ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  const int64_t unit = vec ? 16 : es;
  const int64_t per_row = row_bytes / unit, total = m * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row, c = i - r * per_row;
    const int64_t soff = r * ld_src * es + c * unit;
    const int64_t off = (r * g.ld + g.col0) * es + c * unit;
    if (vec) {
      const uint4 v = *reinterpret_cast<const uint4 *>(src + soff);
      for (int p = 0; p < g.world; p++)
        if (p != skip) *reinterpret_cast<uint4 *>(static_cast<char *>(g.dst[p]) + off) = v;
    } else if (es == 4) {
      const uint32_t v = *reinterpret_cast<const uint32_t *>(src + soff);
      for (int p = 0; p < g.world; p++)
        if (p != skip) *reinterpret_cast<uint32_t *>(static_cast<char *>(g.dst[p]) + off) = v;
    } else {
      const uint16_t v = *reinterpret_cast<const uint16_t *>(src + soff);
      for (int p = 0; p < g.world; p++)
        if (p != skip) *reinterpret_cast<uint16_t *>(static_cast<char *>(g.dst[p]) + off) = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) gather_publish_and_wait(g);
}

// One warp: lane p awaits, bounded, rank p's epoch of the gathers this rank has published so far (every rank issues
// the same sequence of gathers, so the peers' counts reach this rank's).
__global__ void __launch_bounds__(32) gather_wait_kernel(GatherArgs g) {
  const int lane = threadIdx.x & 31;
  const unsigned int epoch = g.ctl[0];
  if (g.ctl[3]) return; // a peer was late before: reported once, not awaited again
  if (lane < g.world && lane != g.rank) gather_await_peer(g, epoch, lane);
}

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline char *slot_ptr(const xnq_comm *c, int r, int slot) { return static_cast<char *>(c->peer[r]) + FLAG_BYTES + (size_t)slot * c->slot_bytes; }

} // namespace
} // namespace xnq

namespace xnq {
int comm_fill_wait(const xnq_comm *c, NormArgs *na) {
  if (!c->connected) return fail(XNQ_ERR_UNSUPPORTED, "comm is not connected to its peers");
  na->wait_ctl = c->ctl;
  na->wait_row = reinterpret_cast<const unsigned int *>(c->region);
  na->wait_world = c->world, na->wait_rank = c->rank;
  return XNQ_OK;
}
} // namespace xnq

using namespace xnq;

extern "C" {

int xnq_comm_create(int rank, int world, size_t slot_bytes, int nslots, xnq_comm **out) {
  clear_error();
  if (!out) return fail(XNQ_ERR_NULL, "comm_create: out is NULL");
  *out = nullptr;
  if (world < 1 || world > XNQ_MAX_RANKS || rank < 0 || rank >= world) return fail(XNQ_ERR_SHAPE, "comm_create: rank %d of %d (at most %d ranks)", rank, world, XNQ_MAX_RANKS);
  if (nslots < 2 || nslots > 64) return fail(XNQ_ERR_SIZE, "comm_create: %d slots; consecutive gathers must alternate between at least 2 (at most 64)", nslots);
  if (slot_bytes == 0) return fail(XNQ_ERR_SIZE, "comm_create: slot_bytes is 0");
  xnq_comm *c = new xnq_comm();
  std::memset(c, 0, sizeof(*c));
  c->rank = rank, c->world = world, c->nslots = nslots, c->last_slot = -1;
  c->slot_bytes = (slot_bytes + 255) & ~(size_t)255;
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaMalloc(&c->region, FLAG_BYTES + c->slot_bytes * nslots);
  if (e == cudaSuccess) e = cudaMemset(c->region, 0, FLAG_BYTES + c->slot_bytes * nslots);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&c->ctl), 64);
  if (e == cudaSuccess) e = cudaMemset(c->ctl, 0, 64);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (c->region) cudaFree(c->region);
    if (c->ctl) cudaFree(c->ctl);
    delete c;
    return fail(XNQ_ERR_CUDA, "comm_create: %s", cudaGetErrorString(e));
  }
  c->peer[rank] = c->region;
  c->connected = world == 1;
  *out = c;
  return XNQ_OK;
}

int xnq_comm_ipc_handle(const xnq_comm *c, void *handle64) {
  clear_error();
  if (!c || !handle64) return fail(XNQ_ERR_NULL, "comm_ipc_handle: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == XNQ_IPC_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  XNQ_CUDA(cudaIpcGetMemHandle(&h, c->region));
  std::memcpy(handle64, &h, sizeof(h));
  return XNQ_OK;
}

int xnq_comm_connect(xnq_comm *c, const void *handles) {
  clear_error();
  if (!c || !handles) return fail(XNQ_ERR_NULL, "comm_connect: NULL argument");
  if (c->connected) return c->world == 1 ? XNQ_OK : fail(XNQ_ERR_UNSUPPORTED, "comm_connect: already connected");
  for (int p = 0; p < c->world; p++) {
    if (p == c->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const char *>(handles) + (size_t)p * XNQ_IPC_HANDLE_BYTES, sizeof(h));
    XNQ_CUDA(cudaIpcOpenMemHandle(&c->peer[p], h, cudaIpcMemLazyEnablePeerAccess));
  }
  c->connected = true;
  return XNQ_OK;
}

int xnq_comm_slot(const xnq_comm *c, int slot, void **ptr, size_t *bytes) {
  clear_error();
  if (!c || !ptr) return fail(XNQ_ERR_NULL, "comm_slot: NULL argument");
  if (slot < 0 || slot >= c->nslots) return fail(XNQ_ERR_SIZE, "comm_slot: slot %d of %d", slot, c->nslots);
  *ptr = slot_ptr(c, c->rank, slot);
  if (bytes) *bytes = c->slot_bytes;
  return XNQ_OK;
}

int xnq_comm_status(const xnq_comm *c, unsigned int *late_peers) {
  clear_error();
  if (!c || !late_peers) return fail(XNQ_ERR_NULL, "comm_status: NULL argument");
  XNQ_CUDA(cudaMemcpy(late_peers, c->ctl + 3, sizeof(unsigned int), cudaMemcpyDeviceToHost));
  return XNQ_OK;
}

int xnq_comm_set_deferred(xnq_comm *c, int deferred) {
  clear_error();
  if (!c) return fail(XNQ_ERR_NULL, "comm_set_deferred: comm is NULL");
  c->deferred = deferred ? 1 : 0;
  return XNQ_OK;
}

int xnq_comm_wait(xnq_comm *c, void *stream) {
  clear_error();
  if (!c) return fail(XNQ_ERR_NULL, "comm_wait: comm is NULL");
  if (!c->connected) return fail(XNQ_ERR_UNSUPPORTED, "comm_wait: comm is not connected to its peers");
  if (c->world == 1) return XNQ_OK;
  GatherArgs g{};
  for (int p = 0; p < c->world; p++) g.flag[p] = reinterpret_cast<unsigned int *>(c->peer[p]) + c->rank;
  g.ctl = c->ctl, g.world = c->world, g.rank = c->rank;
  gather_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(g);
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  return XNQ_OK;
}

int xnq_comm_free(xnq_comm *c) {
  clear_error();
  if (!c) return XNQ_OK;
  for (int p = 0; p < c->world; p++)
    if (p != c->rank && c->peer[p]) cudaIpcCloseMemHandle(c->peer[p]);
  cudaFree(c->region);
  cudaFree(c->ctl);
  delete c;
  return XNQ_OK;
}

int xnq_comm_gather(xnq_comm *c, int slot, const void *src, int elem_dtype, int64_t m, int64_t n_local, int64_t ld_src, void *stream, void **y_out) {
  clear_error();
  if (!c) return fail(XNQ_ERR_NULL, "comm_gather: comm is NULL");
  if (!c->connected) return fail(XNQ_ERR_UNSUPPORTED, "comm_gather: comm is not connected to its peers");
  if (slot < 0 || slot >= c->nslots) return fail(XNQ_ERR_SIZE, "comm_gather: slot %d of %d", slot, c->nslots);
  if (slot == c->last_slot) return fail(XNQ_ERR_UNSUPPORTED, "comm_gather: slot %d was written by the previous gather; alternate slots", slot);
  if (!is_float_dtype(elem_dtype)) return fail(XNQ_ERR_DTYPE, "comm_gather: element dtype %d is not f32/f16/bf16", elem_dtype);
  if (m < 1 || n_local < 1 || ld_src < n_local) return fail(XNQ_ERR_SHAPE, "comm_gather: m = %lld, n_local = %lld, ld_src = %lld", (long long)m, (long long)n_local, (long long)ld_src);
  if (!src) return fail(XNQ_ERR_NULL, "comm_gather: src is NULL");
  const size_t es = type_size(elem_dtype);
  if (!aligned_to(src, es)) return fail(XNQ_ERR_ALIGN, "comm_gather: src is not aligned to its element size");
  const int64_t nt = n_local * c->world;
  if ((size_t)m * (size_t)nt * es > c->slot_bytes)
    return fail(XNQ_ERR_SIZE, "comm_gather: [%lld, %lld] output needs %zu bytes, slots have %zu", (long long)m, (long long)nt, (size_t)m * nt * es, c->slot_bytes);
  GatherArgs g{};
  for (int p = 0; p < c->world; p++) {
    g.dst[p] = slot_ptr(c, p, slot);
    g.flag[p] = reinterpret_cast<unsigned int *>(c->peer[p]) + c->rank;
  }
  g.ctl = c->ctl, g.world = c->world, g.rank = c->rank, g.col0 = n_local * c->rank, g.ld = nt, g.cta_fence_gpu = gather_cta_fence_scope(), g.defer_wait = c->deferred;
  const int64_t units = m * n_local;
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(296, (units + 1023) / 1024));
  gather_push_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(g, src, ld_src, m, n_local, (int)es, -1);
  XNQ_CUDA(cudaGetLastError());
  count_launch();
  c->last_slot = slot;
  if (y_out) *y_out = slot_ptr(c, c->rank, slot);
  return XNQ_OK;
}

int xnq_matmul_t_gather(const xnq_weight *w, xnq_comm *c, int slot, int layout, const void *x, int x_dtype, int64_t m, int64_t ldx, int y_dtype,
                        void *workspace, size_t ws_bytes, void *stream, void **y_out) {
  clear_error();
  if (!w || !c) return fail(XNQ_ERR_NULL, "matmul_t_gather: weight or comm is NULL");
  if (!c->connected) return fail(XNQ_ERR_UNSUPPORTED, "matmul_t_gather: comm is not connected to its peers");
  if (slot < 0 || slot >= c->nslots) return fail(XNQ_ERR_SIZE, "matmul_t_gather: slot %d of %d", slot, c->nslots);
  if (slot == c->last_slot) return fail(XNQ_ERR_UNSUPPORTED, "matmul_t_gather: slot %d was written by the previous gather; alternate slots", slot);
  if (!is_float_dtype(y_dtype)) return fail(XNQ_ERR_DTYPE, "matmul_t_gather: output dtype %d is not f32/f16/bf16", y_dtype);
  if (m < 1) return fail(XNQ_ERR_SHAPE, "matmul_t_gather: m = %lld (every rank must take part in every gather)", (long long)m);
  if (layout != XNQ_GATHER_COLUMNS && layout != XNQ_GATHER_PARTS) return fail(XNQ_ERR_UNSUPPORTED, "matmul_t_gather: layout %d", layout);
  // columns: this rank's rows of an N-sharded weight land at their place in [m, n_total];
  // parts:   every rank holds a whole-N weight (its K-shard) and its [m, n] result becomes block `rank` of [m, world * n]
  const int64_t n = w->v.n, nt = layout == XNQ_GATHER_COLUMNS ? w->n_total : n * c->world;
  const int64_t col0 = layout == XNQ_GATHER_COLUMNS ? w->row0 : n * c->rank;
  const size_t es = type_size(y_dtype);
  if ((size_t)m * (size_t)nt * es > c->slot_bytes)
    return fail(XNQ_ERR_SIZE, "matmul_t_gather: [%lld, %lld] output needs %zu bytes, slots have %zu", (long long)m, (long long)nt, (size_t)m * nt * es, c->slot_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  GatherArgs g{};
  for (int p = 0; p < c->world; p++) {
    g.dst[p] = slot_ptr(c, p, slot);
    g.flag[p] = reinterpret_cast<unsigned int *>(c->peer[p]) + c->rank;
  }
  g.ctl = c->ctl, g.world = c->world, g.rank = c->rank, g.col0 = col0, g.ld = nt, g.cta_fence_gpu = gather_cta_fence_scope(), g.defer_wait = c->deferred;
  char *local = slot_ptr(c, c->rank, slot);
  int rc;
  if (m == 1 && matvec_tma_enabled() && matvec_tma_supported(w->v, 1)) {
    if (x_dtype == XNQ_ACT_IMAGE) {
      if (!x || (reinterpret_cast<uintptr_t>(x) & 255)) return fail(XNQ_ERR_ALIGN, "matmul_t_gather: the activation image must be non-NULL and 256-byte aligned");
    } else if ((rc = check_activations("matmul_t_gather", x, x_dtype, m, w->v.k, ldx)) != XNQ_OK) {
      return rc;
    }
    const void *xin = x;
    int xin_dtype = x_dtype;
    if (x_dtype != XNQ_ACT_IMAGE && matvec_tma_wants_image(w->v)) { // long rows: quantized into the workspace first
      const size_t need = act_workspace_bytes(1, w->v.k, act_dtype_for(w->v.dtype));
      if (!workspace || ws_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return fail(XNQ_ERR_SIZE, "matmul_t_gather: k = %lld needs a 256-byte aligned workspace of %zu bytes", (long long)w->v.k, need);
      const ActView a = act_view(workspace, 1, w->v.k, act_dtype_for(w->v.dtype));
      if ((rc = launch_quantize_act_planar(a, x, x_dtype, ldx, s)) != XNQ_OK) return rc;
      xin = workspace;
      xin_dtype = XNQ_ACT_IMAGE;
    }
    rc = launch_matvec_tma(w->v, xin, xin_dtype, nullptr, y_dtype, s, &g); // stores go to every rank's slot from inside the kernel
    if (rc != XNQ_OK) return rc;
  } else {
    rc = xnq_matmul_t(w, x, x_dtype, m, ldx, local + (size_t)col0 * es, y_dtype, nt, workspace, ws_bytes, s);
    if (rc != XNQ_OK) return rc;
    const int64_t units = m * n;
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(296, (units + 1023) / 1024));
    gather_push_kernel<<<grid, 256, 0, s>>>(g, local + (size_t)col0 * es, nt, m, n, (int)es, c->rank);
    XNQ_CUDA(cudaGetLastError());
    count_launch();
  }
  c->last_slot = slot;
  if (y_out) *y_out = local;
  return XNQ_OK;
}

} // extern "C"
