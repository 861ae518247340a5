// C++ host layer over the xnq C ABI, shaped like xn-core's quantized operator API.
//
//   reference (Rust)                                             here
//   GgmlDType                xn-core/src/quantized/mod.rs:77-196  xnq::GgmlDType, type_size, block_size
//   QTensor                  quantized/mod.rs:27-340              xnq::QTensor      (host blocks + shape)
//   Q8Tensor                 cuda_backend/q8.rs:26-157            xnq::QCudaTensor  (device weight)
//   Q8Linear / QLinear       q8.rs:160-185, mod.rs:342-406        xnq::QCudaLinear
//   Q8<T>: BackendQ          q8.rs:187-224, lib.rs:141-156        xnq::Q40 / Q41 / Q50 / Q51 / Q80 / Q2K / Q3K / Q4K / Q5K / Q6K
//
// xn's Tensor<T, Device> does not exist on this side of the ABI, so device tensors are a pointer, a
// dtype and their dimensions. Errors are exceptions carrying the ABI's status code and message, the
// way the Rust side turns them into xn::Error. Header-only; link libxnq and the CUDA runtime.
#pragma once

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "xnq.h"

namespace xnq {

enum class GgmlDType : int {
  F32 = XNQ_F32, F16 = XNQ_F16, Q4_0 = XNQ_Q4_0, Q4_1 = XNQ_Q4_1, Q5_0 = XNQ_Q5_0, Q5_1 = XNQ_Q5_1, Q8_0 = XNQ_Q8_0, Q8_1 = XNQ_Q8_1,
  Q2K = XNQ_Q2K, Q3K = XNQ_Q3K, Q4K = XNQ_Q4K, Q5K = XNQ_Q5K, Q6K = XNQ_Q6K, Q8K = XNQ_Q8K, BF16 = XNQ_BF16
};

inline size_t type_size(GgmlDType d) { return (size_t)xnq_type_size((int)d); }   // mod.rs:160-179
inline size_t block_size(GgmlDType d) { return (size_t)xnq_block_size((int)d); } // mod.rs:182-195
inline const char *name(GgmlDType d) {
  switch (d) {
    case GgmlDType::F32: return "F32";
    case GgmlDType::F16: return "F16";
    case GgmlDType::BF16: return "BF16";
    case GgmlDType::Q4_0: return "Q4_0";
    case GgmlDType::Q4_1: return "Q4_1";
    case GgmlDType::Q5_0: return "Q5_0";
    case GgmlDType::Q5_1: return "Q5_1";
    case GgmlDType::Q8_0: return "Q8_0";
    case GgmlDType::Q8_1: return "Q8_1";
    case GgmlDType::Q2K: return "Q2K";
    case GgmlDType::Q3K: return "Q3K";
    case GgmlDType::Q4K: return "Q4K";
    case GgmlDType::Q5K: return "Q5K";
    case GgmlDType::Q6K: return "Q6K";
    case GgmlDType::Q8K: return "Q8K";
  }
  return "?";
}

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};
inline void check(int rc) {
  if (rc != XNQ_OK) throw Error(rc, xnq_last_error());
}
[[noreturn]] inline void bail(const std::string &m) { throw Error(XNQ_ERR_SHAPE, m); }

inline std::string dims_string(const std::vector<int64_t> &d) {
  std::string s = "[";
  for (size_t i = 0; i < d.size(); i++) s += (i ? ", " : "") + std::to_string(d[i]);
  return s + "]";
}

// Quantized blocks in host memory with a shape; data() is the canonical GGUF byte image (mod.rs:330-332).
class QTensor {
 public:
  QTensor(std::vector<uint8_t> blocks, std::vector<int64_t> shape, GgmlDType dtype) : data_(std::move(blocks)), shape_(std::move(shape)), dtype_(dtype) {
    if (shape_.empty()) bail("scalar tensor cannot be quantized " + dims_string(shape_));                                  // mod.rs:264-266
    const size_t bs = block_size(dtype_);
    if (bs == (size_t)-1 || bs == 0) bail(std::string("unsupported quantized dtype ") + name(dtype_));
    if (shape_.back() % (int64_t)bs != 0)
      bail("quantized tensor must have their last dim divisible by block size " + dims_string(shape_) + " " + std::to_string(bs)); // mod.rs:267-272
    int64_t elems = 1;
    for (int64_t d : shape_) elems *= d;
    const size_t want = (size_t)elems / bs * type_size(dtype_);
    if (data_.size() != want) bail(std::string(name(dtype_)) + " " + dims_string(shape_) + " wants " + std::to_string(want) + " bytes of blocks, got " + std::to_string(data_.size()));
  }
  GgmlDType dtype() const { return dtype_; }
  size_t rank() const { return shape_.size(); }
  const std::vector<int64_t> &shape() const { return shape_; }
  size_t storage_size_in_bytes() const { return data_.size(); }
  const std::vector<uint8_t> &data() const { return data_; }

 private:
  std::vector<uint8_t> data_;
  std::vector<int64_t> shape_;
  GgmlDType dtype_;
};

// A (n, k) quantized weight, or an N-shard of one, resident on the current CUDA device.
class QCudaTensor {
 public:
  // Take GGUF blocks as they are (Q8Tensor::from_q8_0, q8.rs:60-85).
  static QCudaTensor from_qtensor(const QTensor &qt, void *stream = nullptr, int shard_rank = 0, int shard_count = 1) {
    if (qt.rank() != 2) bail("cuda quantized: expected a 2-d weight, got shape " + dims_string(qt.shape()));
    xnq_weight *h = nullptr;
    check(xnq_weight_upload((int)qt.dtype(), qt.data().data(), qt.data().size(), qt.shape()[0], qt.shape()[1], shard_rank, shard_count, stream, &h));
    return QCudaTensor(h);
  }
  QCudaTensor(QCudaTensor &&o) noexcept { *this = std::move(o); }
  QCudaTensor &operator=(QCudaTensor &&o) noexcept {
    if (this != &o) {
      release();
      h_ = o.h_, dtype_ = o.dtype_, n_total_ = o.n_total_, n_ = o.n_, row0_ = o.row0_, k_ = o.k_;
      o.h_ = nullptr;
    }
    return *this;
  }
  QCudaTensor(const QCudaTensor &) = delete;
  QCudaTensor &operator=(const QCudaTensor &) = delete;
  ~QCudaTensor() { release(); }

  GgmlDType dtype() const { return dtype_; }
  std::pair<int64_t, int64_t> shape() const { return {n_, k_}; } // rows held here, k
  int64_t n_total() const { return n_total_; }
  int64_t row0() const { return row0_; }
  const xnq_weight *handle() const { return h_; }

  // Canonical GGUF bytes of the held rows (QuantizedType::raw_data contract, mod.rs:206-214).
  std::vector<uint8_t> data(void *stream = nullptr) const {
    std::vector<uint8_t> out((size_t)n_ * (size_t)(k_ / (int64_t)block_size(dtype_)) * type_size(dtype_));
    check(xnq_weight_canonical_bytes(h_, out.data(), out.size(), stream));
    return out;
  }
  // Dense (n, k) copy into device memory `dst` (Q8Tensor::dequantize, q8.rs:94-113).
  void dequantize(void *dst, GgmlDType out_dtype, void *stream = nullptr) const { check(xnq_weight_dequantize(h_, (int)out_dtype, dst, stream)); }
  size_t workspace_bytes(int64_t max_m) const { return xnq_matmul_workspace_bytes(h_, max_m); }
  // `lhs @ self^T`: lhs is m rows of k (row stride ldx elements), y is m rows of n (q8.rs:116-157).
  void matmul_t(const void *x, GgmlDType x_dtype, int64_t m, int64_t ldx, void *y, GgmlDType y_dtype, int64_t ldy, void *workspace, size_t ws_bytes,
                void *stream = nullptr) const {
    check(xnq_matmul_t(h_, x, (int)x_dtype, m, ldx, y, (int)y_dtype, ldy, workspace, ws_bytes, stream));
  }
  // QLinear::forward on host tensors (mod.rs:352-384).
  void forward_host(const float *x, int64_t m, const float *bias, float *y, void *stream = nullptr) { check(xnq_linear_forward_host(h_, x, m, bias, y, stream)); }

 private:
  explicit QCudaTensor(xnq_weight *h) : h_(h) {
    int dt = 0;
    size_t bytes = 0;
    check(xnq_weight_info(h_, &dt, &n_total_, &n_, &row0_, &k_, &bytes));
    dtype_ = (GgmlDType)dt;
  }
  void release() {
    if (h_) xnq_weight_free(h_);
    h_ = nullptr;
  }
  xnq_weight *h_ = nullptr;
  GgmlDType dtype_ = GgmlDType::F32;
  int64_t n_total_ = 0, n_ = 0, row0_ = 0, k_ = 0;
};

// A linear layer with GGUF-quantized weights on the device and an optional f32 bias in host memory
// (Q8Linear, q8.rs:160-185). forward takes the flattened leading dimensions as m.
class QCudaLinear {
 public:
  explicit QCudaLinear(QCudaTensor weight, std::vector<float> bias = {}) : weight_(std::move(weight)), bias_(std::move(bias)) {
    if (!bias_.empty() && (int64_t)bias_.size() != weight_.shape().first) bail("bias length does not match out_features");
  }
  const QCudaTensor &weight() const { return weight_; }
  // xs dims as in the reference: rank >= 2, last dim == k (mod.rs:363-370); returns the output dims.
  std::vector<int64_t> forward_host(const float *xs, const std::vector<int64_t> &dims, float *out, void *stream = nullptr) {
    if (dims.size() < 2) bail("input tensor has only one dimension " + dims_string(dims));
    const auto [n, k] = weight_.shape();
    if (dims.back() != k) bail("input tensor " + dims_string(dims) + " incompatible with " + dims_string({n, k}));
    int64_t m = 1;
    for (size_t i = 0; i + 1 < dims.size(); i++) m *= dims[i];
    weight_.forward_host(xs, m, bias_.empty() ? nullptr : bias_.data(), out, stream);
    std::vector<int64_t> od(dims.begin(), dims.end() - 1);
    od.push_back(n);
    return od;
  }

 private:
  QCudaTensor weight_;
  std::vector<float> bias_;
};

// BackendQ for the CUDA device with one GGML weight format (lib.rs:141-156). linear_load's branch that
// takes a file's blocks as they are (q8.rs:203-213): dtype and shape must match; weight only, no bias.
template <GgmlDType D>
struct BackendQ {
  static constexpr GgmlDType DTYPE = D;
  static QCudaLinear linear_from_qtensor(const QTensor &qt, int64_t in_features, int64_t out_features, void *stream = nullptr, int shard_rank = 0,
                                         int shard_count = 1) {
    if (qt.dtype() != D) bail(std::string("cuda ") + name(D) + ": expected a " + name(D) + " tensor, got " + name(qt.dtype()));
    if (qt.rank() != 2 || qt.shape()[0] != out_features || qt.shape()[1] != in_features)
      bail(std::string("cuda ") + name(D) + ": weight is " + dims_string(qt.shape()) + ", expected " + dims_string({out_features, in_features}));
    return QCudaLinear(QCudaTensor::from_qtensor(qt, stream, shard_rank, shard_count));
  }
};
using Q40 = BackendQ<GgmlDType::Q4_0>;
using Q80 = BackendQ<GgmlDType::Q8_0>;
using Q4K = BackendQ<GgmlDType::Q4K>;
using Q6K = BackendQ<GgmlDType::Q6K>;
// the remaining weight formats the reference instantiates (mod.rs:444-455): held as the file's blocks, one plain kernel each
using Q41 = BackendQ<GgmlDType::Q4_1>;
using Q50 = BackendQ<GgmlDType::Q5_0>;
using Q51 = BackendQ<GgmlDType::Q5_1>;
using Q2K = BackendQ<GgmlDType::Q2K>;
using Q3K = BackendQ<GgmlDType::Q3K>;
using Q5K = BackendQ<GgmlDType::Q5K>;

} // namespace xnq
