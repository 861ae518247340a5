/*
 * xnq: B200-native (sm_100a) GGUF block-quantized matmul, C ABI.
 *
 * This is the boundary an xn-core build binds over FFI (the way xn-flash-attn binds `run_mha`,
 * xn-flash-attn/src/ffi.rs:3-57) to put Q4_0 / Q8_0 / Q4_K / Q6_K linears on the GPU behind its
 * existing `BackendQ` / `ModuleT` operator API (xn-core/src/lib.rs:123-156). Plain pointers and
 * sizes only; no C++ or torch types. Every function returns XNQ_OK (0) or a negative xnq_status
 * and never throws or aborts; xnq_last_error() gives the message for the calling thread.
 * All shape / size / alignment validation happens before anything is enqueued.
 *
 * Streams: `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream). Compute
 * entries only enqueue on it and return; they neither allocate nor synchronize, so they may be
 * recorded into a CUDA graph once xnq_init() has run for the device.
 *
 * There is no CPU fallback anywhere behind this header.
 */
#ifndef XNQ_H
#define XNQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XNQ_VERSION 1

typedef enum xnq_status {
  XNQ_OK = 0,
  XNQ_ERR_NULL = -1,        /* a required pointer is NULL */
  XNQ_ERR_DTYPE = -2,       /* unsupported GGML / activation dtype */
  XNQ_ERR_SHAPE = -3,       /* k not a multiple of the block, negative sizes, shard mismatch */
  XNQ_ERR_ALIGN = -4,       /* pointer or leading dimension not aligned as documented */
  XNQ_ERR_SIZE = -5,        /* byte count / workspace too small, or over a documented maximum */
  XNQ_ERR_CUDA = -6,        /* a CUDA runtime call failed; message carries cudaGetErrorString */
  XNQ_ERR_COMM = -7,        /* multi-GPU exchange failed or timed out */
  XNQ_ERR_UNSUPPORTED = -8, /* valid request this build cannot serve (e.g. device is not sm_100) */
} xnq_status;

/* dtype codes are the GGML ids (GgmlDType::to_u32, xn-core/src/quantized/mod.rs:119-137) */
enum {
  XNQ_F32 = 0,
  XNQ_F16 = 1,
  XNQ_Q4_0 = 2,
  XNQ_Q4_1 = 3,
  XNQ_Q5_0 = 6,
  XNQ_Q5_1 = 7,
  XNQ_Q8_0 = 8,
  XNQ_Q8_1 = 9, /* activation blocks only */
  XNQ_Q2K = 10,
  XNQ_Q3K = 11,
  XNQ_Q4K = 12,
  XNQ_Q5K = 13,
  XNQ_Q6K = 14,
  XNQ_Q8K = 15, /* activation blocks only */
  XNQ_BF16 = 30,
};
/* Weight formats: Q4_0, Q8_0, Q4_K, Q6_K (the formats of the benchmark configurations) have their own device layouts and
 * HBM-streaming / tensor-core kernels. Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K are held as the file's blocks and served by one
 * plain kernel each for to_float and matmul (same results contract; no activation image, gather or static entry). */

/* An immutable quantized [n, k] weight (or an N-shard of one) resident in device memory.
 * Replaces Q8Tensor (xn-core/src/cuda_backend/q8.rs:26-33) and the missing QStorage::Cuda variant
 * (xn-core/src/quantized/mod.rs:32-34). The weight is immutable after upload: every entry that takes a
 * `const xnq_weight *` may be called on one handle from several host threads at once. The two entries that
 * take a non-const handle (xnq_linear_forward_host, xnq_weight_reserve_host_staging) use staging buffers
 * owned by the handle and must not run concurrently with each other on the same handle. */
typedef struct xnq_weight xnq_weight;
typedef struct xnq_comm xnq_comm; /* a rank's end of the kernel-side output exchange, see xnq_comm_create */

/* Message of the last failure on the calling thread ("" if none). Replaces the xn::Error text a
 * Rust caller builds with bail! (xn-core/src/error.rs:153-164). */
const char *xnq_last_error(void);
int xnq_version(void);

/* Loads every kernel of the library on `device`, raises their shared-memory limits and checks the
 * device is compute capability 10.x. Call once per device before the first stream capture.
 * Stands in for the lazy PTX module load in Device::get_func (cuda_backend/mod.rs:311-403). */
int xnq_init(int device);

/* bytes per block / elements per block of a GGML dtype (GgmlDType::type_size / block_size,
 * quantized/mod.rs:160-195); -1 for a dtype this library does not handle */
int xnq_type_size(int ggml_dtype);
int xnq_block_size(int ggml_dtype);

/* Upload. `blocks` is the canonical GGUF byte image of the FULL [n, k] tensor, in host or device memory
 * (what QTensor::data() returns, quantized/mod.rs:330-332), nbytes = n * (k / block) * type_size.
 * With shard_count G > 1 only rows [r*n/G, (r+1)*n/G) are uploaded (n must divide by G).
 * The device layout may differ from GGUF (the reference's own Q8_0 upload re-lays out too,
 * q8.rs:9-11,78-91); xnq_weight_canonical_bytes gives the canonical bytes back exactly.
 * Synchronizes `stream` before returning. Replaces Q8Tensor::from_q8_0 (q8.rs:60-85). */
int xnq_weight_upload(int ggml_dtype, const void *blocks, size_t nbytes, int64_t n, int64_t k,
                      int shard_rank, int shard_count, void *stream, xnq_weight **out);
/* Same, but `blocks` holds only rows [row0, row0 + n_rows) of an [n_total, k] tensor. */
int xnq_weight_upload_rows(int ggml_dtype, const void *blocks, size_t nbytes, int64_t n_total,
                           int64_t k, int64_t row0, int64_t n_rows, void *stream, xnq_weight **out);
/* Replaces Drop of Q8Tensor's CudaSlices. NULL is accepted. */
int xnq_weight_free(xnq_weight *w);
/* Any out pointer may be NULL. n_local / row0 describe the shard held (QTensor::shape / dtype,
 * quantized/mod.rs:305-315). */
int xnq_weight_info(const xnq_weight *w, int *ggml_dtype, int64_t *n_total, int64_t *n_local,
                    int64_t *row0, int64_t *k, size_t *device_bytes);

/* Dense [n_local, k] row-major copy of the weight in out_dtype (XNQ_F32 / XNQ_F16 / XNQ_BF16);
 * f32 output is bit-identical to GgmlType::to_float (k_quants.rs:213-233,618-634,1475-1503,
 * 1874-1904). Replaces Q8Tensor::dequantize (q8.rs:94-113). dst is device memory. */
int xnq_weight_dequantize(const xnq_weight *w, int out_dtype, void *dst, void *stream);
/* Canonical GGUF bytes of the held rows into HOST memory (QTensor::data contract,
 * quantized/mod.rs:206-214). Synchronizes `stream`. */
int xnq_weight_canonical_bytes(const xnq_weight *w, void *host_dst, size_t nbytes, void *stream);

/* Activations quantized ahead of the matmul. The reference quantizes the activations inside every
 * matmul call (quantize_lhs, k_quants.rs:2015-2026); when several linears read the same input, or the
 * producer of the input can quantize it as it writes it (xnq_add_rmsnorm, xnq_swiglu), that work is done
 * once: an "activation image" holds m rows of Q8_0 or Q8_K codes, block scales and 16-element sums in the
 * planar layout the kernels read, and is passed to xnq_matmul_t / xnq_matmul_t_gather as x with
 * x_dtype = XNQ_ACT_IMAGE (m <= 16; ldx and the workspace are ignored). The bytes are those the in-call
 * quantizer produces, so results are identical. act_dtype is XNQ_Q8_0 for Q4_0 / Q8_0 weights and XNQ_Q8K
 * for Q4_K / Q6_K weights. The image must be 256-byte aligned. */
#define XNQ_ACT_IMAGE 100
/* A second form for batches of 2..64 rows on Q4_K weights: the rows quantized to Q8_K (the same codes, scales and sums) in the
 * layout the integer tensor-core kernel reads, so that xnq_matmul_t(.., x_dtype = XNQ_ACT_OPERAND, ..) is ONE kernel (with
 * float rows or an XNQ_ACT_IMAGE it launches a kernel of its own first that quantizes / re-lays the activations). Written by
 * xnq_add_rmsnorm and xnq_swiglu with act_dtype = XNQ_ACT_OPERAND. xnq_act_operand_bytes(m, k): size (k a multiple of 256,
 * m <= 64; 0 otherwise). The buffer is 256-byte aligned, belongs to one (m, k), and must be zeroed once after allocation
 * (rows m.. of the padded batch and the ticket words are never written by a producer). Results are bit for bit those of the
 * other input forms. One matmul at a time may read an image (its ticket words are in the image). */
#define XNQ_ACT_OPERAND 101
size_t xnq_act_operand_bytes(int64_t m, int64_t k);
size_t xnq_act_image_bytes(int act_dtype, int64_t m, int64_t k);
int xnq_quantize_act_image(int act_dtype, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx,
                           void *image, void *stream);

/* QTensor::quantize_f32 / QLinear::from_linear for a weight that already lives on the device
 * (quantized/mod.rs:290-297, 398-405): x_dev is a dense f32 [n, k] matrix, blocks_dev receives
 * n * k / block GGUF blocks in canonical byte order, bit-identical to the reference's host
 * quantizers (BlockQ4_0 / BlockQ8_0 / BlockQ4K / BlockQ6K ::from_float, k_quants.rs:235-270,
 * 636-661, 1418-1473, 1801-1871 with utils.rs:65-254). Both pointers 16-byte aligned. Feed the
 * result to xnq_weight_upload, which accepts host or device memory for `blocks`. */
int xnq_quantize_weight(int ggml_dtype, const float *x_dev, int64_t n, int64_t k, void *blocks_dev, void *stream);

/* Quantize activations x [m, k] (row stride ldx elements, x_dtype F32/F16/BF16, device memory) to
 * canonical activation blocks in device memory: act_dtype XNQ_Q8_0 gives m*k/32 BlockQ8_0 (34 B),
 * XNQ_Q8K gives m*k/256 BlockQ8K (292 B, bsums included). Byte-identical to
 * BlockQ8_0::from_float / BlockQ8K::from_float (k_quants.rs:636-661, 1942-1979), which is what
 * quantize_lhs runs per row (k_quants.rs:2015-2026). */
int xnq_quantize_act(int act_dtype, const void *x, int x_dtype, int64_t m, int64_t k, int64_t ldx,
                     void *dst_blocks, void *stream);

/* Scratch bytes xnq_matmul_t needs for up to max_m activation rows against this weight. */
size_t xnq_matmul_workspace_bytes(const xnq_weight *w, int64_t max_m);

/* y[m, n_local] = x[m, k] . W^T, the quantized matmul of k_quants::matmul (k_quants.rs:1997-2011)
 * = QTensor::matmul_t (quantized/mod.rs:334-339) = Q8Tensor::matmul_t (q8.rs:116-157):
 * activations are quantized to the weight format's VecDotType exactly as the CPU path does, dots
 * use exact integer block sums and f32 accumulation (m <= 16), or tensor-core MMA on the
 * dequantized operands (m > 16).
 *   x, y: device memory, x_dtype / y_dtype in {F32, F16, BF16}; ldx, ldy in elements;
 *   x rows 16-byte aligned; workspace 256-byte aligned, ws_bytes >= xnq_matmul_workspace_bytes.
 * Enqueues on `stream` only; allocates nothing. */
int xnq_matmul_t(const xnq_weight *w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y,
                 int y_dtype, int64_t ldy, void *workspace, size_t ws_bytes, void *stream);

/* A prefetch hint (no counterpart in the reference): names the weight that the calling thread will multiply
 * AFTER its next one-row (m == 1) xnq_matmul_t / xnq_matmul_t_gather call. That next call's kernel then asks for
 * the named weight's bytes to be brought into L2 while it streams its own weight, so HBM stays busy across the
 * launch boundary (a decoder knows its next linear; a loop over layers names layer l + 1 before multiplying layer
 * l). One-shot and per host thread; NULL clears it. Results never depend on it. The named weight must stay
 * alive until that launch has finished; under stream capture the hint is recorded with the launch. */
int xnq_hint_next_weight(const xnq_weight *w);
/* One row, three operators in one launch: x_out[k] = x_in[k] + sum of the `delta_parts` rows of delta ([parts][k], may
 * be NULL with 0 parts), then y[n] = W . quantize(rmsnorm(x_out) * norm_weight). The results are, bit for bit, those of
 * xnq_add_rmsnorm (with an activation image) followed by xnq_matmul_t: every CTA of the matvec forms the normalised,
 * quantized row for itself, one of them writes the new residual. x_out must not be x_in. f32 rows of at most 4096
 * values whose weight the one-row kernel serves; otherwise XNQ_ERR_UNSUPPORTED (call the two operators instead).
 * `await` (may be NULL): the communicator whose slot holds `delta` when the gather that produced it was left
 * un-awaited (xnq_comm_set_deferred): the kernel streams its weight while it awaits, bounded, the peers' epochs, and
 * reads the summands only then.
 * Reference: the rms_norm + linear pairs of a decoder layer, xn-core/src/models/llama.rs:145-216. */
int xnq_matvec_normed(const xnq_weight *w, const float *x_in, const float *delta, int delta_parts, const float *norm_weight,
                      float eps, float *x_out, void *y, int y_dtype, const xnq_comm *await, void *stream);

/* xnq_matmul_t for callers that can neither supply a workspace nor let the library allocate one:
 * hosts whose allocator owns all device memory, steps being recorded into a CUDA graph, plugins under
 * a fixed memory budget. Same arithmetic and tolerance as xnq_matmul_t (exact integer block sums, f32
 * accumulation; the f32 summation order, and so the last bits, can differ from xnq_matmul_t's, which may pick
 * another kernel for the same shape), for 0 <= m <= 16; the quantized-activation scratch is a 128 KiB array built into the library (each GPU
 * that loads the library holds it until the process exits). Rows are taken in passes that fit the
 * array (1.25 bytes per activation element); a request fails with XNQ_ERR_SIZE only when a single
 * row does not fit, i.e. k above about 104,000, or m > 16. It calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 * The first call on a device looks up the array's device address; make that call (or any call of this
 * entry) once per device before starting a stream capture. All calls share the one array: it keeps
 * the previous call's contents (nothing needs clearing, each call rewrites what it reads), and two
 * calls that overlap on the GPU - different streams, or different threads - race on it; callers must
 * order them. This entry has no counterpart in the reference. */
int xnq_matmul_t_static(const xnq_weight *w, const void *x, int x_dtype, int64_t m, int64_t ldx, void *y,
                        int y_dtype, int64_t ldy, void *stream);

/* QLinear::forward on HOST tensors (quantized/mod.rs:352-384): copies x_host [m, k] f32 to the
 * device, runs xnq_matmul_t, adds bias_host[n_local] if non-NULL, copies y back to y_host
 * [m, n_local] and synchronizes. Device staging buffers are owned by the weight handle:
 * xnq_weight_reserve_host_staging(w, max_m) sizes them ahead of time, after which calls with m <= max_m
 * allocate nothing; without it the first call at a larger m allocates (and is refused with
 * XNQ_ERR_UNSUPPORTED if the stream is being captured). One thread at a time per handle.
 * When y_host is page-locked memory (cudaHostAlloc / cudaHostRegister), there is no bias and m <= 16,
 * the kernel stores the result straight into it and the copy back is skipped. */
int xnq_linear_forward_host(xnq_weight *w, const float *x_host, int64_t m, const float *bias_host,
                            float *y_host, void *stream);
/* No counterpart in the reference (its QLinear::forward allocates a fresh Vec per call, quantized/mod.rs:373-376). */
int xnq_weight_reserve_host_staging(xnq_weight *w, int64_t max_m);

/* ---- N-sharded matmul with the output gather done by the kernels (no counterpart in the
 * reference, which runs on one device: cuda_backend/mod.rs:141-167). One process per GPU; rank r of
 * `world` holds weight rows [r*n/G, (r+1)*n/G) (xnq_weight_upload's shard arguments). Each rank owns
 * one device allocation of `nslots` output slots plus a row of epoch words, maps its peers'
 * allocations through CUDA IPC, and the matmul kernel stores its output columns into the same slot
 * of every rank; a one-warp kernel then waits (bounded) until every peer's columns have arrived.
 * Every rank must issue the same sequence of gathers. Works inside a captured CUDA graph. --------- */
#define XNQ_IPC_HANDLE_BYTES 64
/* Allocates this rank's slots on the current device: nslots (2..64) buffers of slot_bytes each. */
int xnq_comm_create(int rank, int world, size_t slot_bytes, int nslots, xnq_comm **out);
/* The XNQ_IPC_HANDLE_BYTES-byte handle of this rank's allocation, to be sent to every peer process
 * by whatever transport the host has (torch.distributed, MPI, a socket). */
int xnq_comm_ipc_handle(const xnq_comm *c, void *handle64);
/* handles: world * XNQ_IPC_HANDLE_BYTES bytes, rank p's handle at p * XNQ_IPC_HANDLE_BYTES (the own
 * entry is ignored). Maps every peer's allocation. The host must put a barrier between the last
 * rank's connect and the first gather. */
int xnq_comm_connect(xnq_comm *c, const void *handles);
/* Local device address and size of a slot. */
int xnq_comm_slot(const xnq_comm *c, int slot, void **ptr, size_t *bytes);
/* y[m, n_total] = x[m, k] @ W^T gathered on every rank, in slot `slot` (row stride n_total elements
 * of y_dtype); *y_out receives the slot's local address. m == 1, k <= 4096: the decode kernel itself
 * stores to every rank; otherwise the local result is pushed by a copy kernel. workspace as for
 * xnq_matmul_t. A slot may be named again once another gather has been issued in between; two
 * consecutive calls on one slot are refused, and a replayed graph must not end on the slot it
 * starts with.
 * layout XNQ_GATHER_COLUMNS: w is this rank's rows of an N-sharded weight; the slot receives [m, n_total].
 * layout XNQ_GATHER_PARTS: every rank holds a whole-N weight (for instance its K-shard of a row-parallel
 * linear, fed with its own slice of the input); the slot receives [m, world * n] with rank r's result in
 * columns [r * n, (r + 1) * n) - the summands of an all-reduce, to be added by the consumer. */
#define XNQ_GATHER_COLUMNS 0
#define XNQ_GATHER_PARTS 1
int xnq_matmul_t_gather(const xnq_weight *w, xnq_comm *c, int slot, int layout, const void *x, int x_dtype,
                        int64_t m, int64_t ldx, int y_dtype, void *workspace, size_t ws_bytes, void *stream,
                        void **y_out);
/* All-gather of a tensor this rank already holds: src is [m, n_local] (row stride ld_src elements of
 * elem_dtype) in local device memory; slot `slot` of every rank receives [m, world * n_local] with
 * rank r's block in columns [r * n_local, (r + 1) * n_local). Same slot rule as above. */
int xnq_comm_gather(xnq_comm *c, int slot, const void *src, int elem_dtype, int64_t m, int64_t n_local,
                    int64_t ld_src, void *stream, void **y_out);
/* Deferred waits. By default the kernel that gathers also waits (bounded) for every peer's columns, so its slot is
 * complete when it retires: every gather is then a barrier between the ranks. With deferred = 1 a gather only
 * publishes this rank's columns and retires; xnq_comm_wait enqueues a one-warp kernel that awaits the peers' columns of
 * ALL gathers issued so far, and must lie between a gather and the first reader of its slot. Several gathers may share
 * one wait (the gathers of a whole step, each into a slot of its own); between two waits a slot may be written once. */
int xnq_comm_set_deferred(xnq_comm *c, int deferred);
int xnq_comm_wait(xnq_comm *c, void *stream);
/* Bit p set: a wait for rank p's columns gave up after 4 s (the results of that gather are not
 * complete). Synchronizes the device. */
int xnq_comm_status(const xnq_comm *c, unsigned int *late_peers);
/* Unmaps the peers and frees the slots. All ranks must have finished their gathers. */
int xnq_comm_free(xnq_comm *c);

/* ---- the operators between the quantized linears of a Llama-style decode step, fused (the callers of
 * the path in xn-core/src/models/llama.rs:145-216, 258-265, 300-320; reference kernels rmsnorm / rope /
 * sdpa in cuda-kernels/reduce.cu). All pointers are device memory, f32 unless stated. ------------- */
/* x[rows, d] += sum over p of delta[rows, p, d] (delta may be NULL; delta_parts >= 1 summands per row,
 * e.g. the per-rank partial results of a row-parallel linear), out = x * rsqrt(mean(x^2) + eps) * weight[d].
 * out may be NULL when only the quantized form is wanted. act_image, when not NULL, receives the activation
 * image (act_dtype XNQ_Q8_0 or XNQ_Q8K) of the normalized rows: exactly what quantizing `out` would give. */
int xnq_add_rmsnorm(float *x, const float *delta, int delta_parts, const float *weight, float eps, float *out,
                    void *act_image, int act_dtype, int64_t rows, int64_t d, void *stream);
/* The two ends of a decode step (llama.rs:300-320, the embedding lookup and the greedy choice of the next token).
 * xnq_embed_rows: x[rows, d] (f32) = table[tokens[r], :] of a bf16 table [vocab, d]; a token outside the table gives zeros
 * and sets status bit 26. It is launched as a plain kernel, never programmatically overlapped: as the first kernel of a
 * step it separates the step from the stores of the step before (xnq_rope_attn_decode relies on that).
 * xnq_argmax_advance: tokens[r] = index of the first largest value of logits[r, 0:n] (torch.argmax's rule; a row without
 * any finite candidate gives 0), then *pos += 1 if pos is not NULL. */
int xnq_embed_rows(const void *table_bf16, const long long *tokens, float *x, int64_t rows, int64_t d, int64_t vocab, void *stream);
int xnq_argmax_advance(const float *logits, int64_t rows, int64_t n, long long *tokens, long long *pos, void *stream);
/* out[rows, f] = silu(gate_up[rows, 0:f]) * gate_up[rows, f:2f]; out / act_image as above. */
int xnq_swiglu(const float *gate_up, float *out, void *act_image, int act_dtype, int64_t rows, int64_t f, void *stream);
/* One new token per sequence: qkv[batch, (heads + 2 kv_heads) * head_dim] -> rotate-half RoPE at
 * position *pos_dev (cos/sin tables [max_seq, head_dim / 2]); q_out[batch, heads, head_dim]; rotated k
 * and plain v are stored as bf16 into k_cache / v_cache [batch, kv_heads, max_seq, head_dim]. */
int xnq_rope_kv_store(const float *qkv, const float *cos_table, const float *sin_table, const long long *pos_dev,
                      float *q_out, void *k_cache, void *v_cache, int64_t batch, int heads, int kv_heads,
                      int head_dim, int64_t max_seq, void *stream);
/* Single-query attention over cache positions 0..*pos_dev: out[batch, heads, head_dim] =
 * softmax(q k^T / sqrt(head_dim)) v with heads / kv_heads query heads per KV head. head_dim 128. The
 * sequence is split over several CTAs per head; `workspace` (xnq_attn_decode_workspace_bytes, zeroed
 * once after allocation, reusable by every later call on the same stream whatever its batch and heads, as long
 * as it is large enough) holds their partial sums. A position outside [0, max_seq) sets a bit of
 * xnq_device_status: xnq_rope_kv_store then stores nothing; this call clamps a position past the cache and
 * writes zeros for a negative one. */
size_t xnq_attn_decode_workspace_bytes(int64_t batch, int heads);
int xnq_attn_decode(const float *q, const void *k_cache, const void *v_cache, const long long *pos_dev, float *out,
                    int64_t batch, int heads, int kv_heads, int head_dim, int64_t max_seq, void *workspace,
                    size_t ws_bytes, void *stream);

/* xnq_rope_kv_store and xnq_attn_decode in one launch: every CTA rotates its own head's q from `qkv`
 * ([batch, (heads + 2 kv_heads) * head_dim] f32, the fused q/k/v projection), the CTAs whose run of positions holds *pos_dev
 * rotate that position's k (and take its v) from `qkv` instead of the cache, and the first query head of every KV head stores
 * them into the caches. Bit for bit the result of the two separate calls; the q_out buffer is not needed.
 * The kernel reads *pos_dev and requests the cache rows below it before it waits for the kernel that produces qkv, so both
 * must be final when that producer STARTS: written in an earlier step, with at least one normally launched kernel or copy
 * (one that is not programmatically dependent, e.g. the step's sampling) in between. A decode loop satisfies this by itself. */
int xnq_rope_attn_decode(const float *qkv, const float *cos_table, const float *sin_table, const long long *pos_dev, void *k_cache,
                         void *v_cache, float *out, int64_t batch, int heads, int kv_heads, int head_dim, int64_t max_seq,
                         void *workspace, size_t ws_bytes, void *stream);

/* Sticky device-side status bits of this library's kernels on the current device (0 = healthy).
 * Bits 0-7, one-row ring kernel: bit 0 a consumer's bounded mbarrier wait expired, bit 1 a producer's, bit 2 a
 * self-check refused an access. Bits 8-15: the same for the fp16 tensor-core kernel. Bits 16-23, integer
 * tensor-core kernel: a wait of the producer (16), a converter (17), the MMA issuer (18), a drain warp (19)
 * expired. Bits 24-25: a decode position outside [0, max_seq) reached xnq_rope_kv_store (24) or
 * xnq_attn_decode (25); bit 26: xnq_embed_rows met a token outside the table. Synchronizes the device.
 * No counterpart in the reference (its kernels never wait on anything). */
int xnq_device_status(unsigned int *bits);
/* When bit 2 of the status is set, a kernel's self-check refused an out-of-range copy or store
 * instead of performing it; this returns what it recorded first: code, block, iteration, offset,
 * bytes, limit (two spare words). Synchronizes the device. No counterpart in the reference. */
int xnq_device_check_record(unsigned long long out[8]);
/* Tuning switches, for A/B measurements: "matvec_tma" (default 1) selects the persistent bulk-copy ring
 * decode kernel for m == 1; 0 forces the plain streaming-load kernel. "matvec_mma" (default 1)
 * selects the integer-MMA kernel for batches of 5..16 rows on Q4_K weights, 0 the dp4a kernel. "imma" (default 1):
 * batches of 2..64 rows on Q4_0 / Q8_0 / Q4_K weights take the tcgen05 integer kernel; 0 sends them to the older
 * kernels. "imma_fold" (default 1): the Q4_K variant of that kernel which folds the sub-block scales into the weight
 * operand is used where it is faster (17..32 rows); 0 never, 2 for every batch of 2..64 rows. "gather_cta_fence"
 * (default 1): scope of the per-CTA fence before the arrival count of a kernel-side gather, 1 = gpu,
 * 0 = system. No counterpart in the reference. */
int xnq_set_option(const char *name, int value);

/* ---- measurement hooks (no counterpart in the reference, which times with CudaEvent::elapsed_ms
 * around whole operators, cuda_backend/mod.rs:76-100) ------------------------------------------ */

/* Kernels this library has launched in this process so far (all threads, all devices). */
uint64_t xnq_launch_count(void);
/* Between xnq_profile_begin and xnq_profile_end every xnq_matmul_t call on the calling thread records
 * a CUDA event pair around its dominant kernel (the matvec or prefill kernel, not the activation
 * quantizer). xnq_profile_end synchronizes those events and returns the summed kernel time and the
 * number of timed launches. At most max_launches pairs are kept; later launches are not timed.
 * Do not use while the stream is being captured into a graph. */
int xnq_profile_begin(int max_launches);
int xnq_profile_end(double *total_ms, int *launches);
#ifdef __cplusplus
}
#endif
#endif /* XNQ_H */
