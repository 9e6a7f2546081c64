// C++ host-side mirror of the operator surface tur uses for quantized linears, over the C ABI
// of turq.h. tur is Rust and reaches this path through candle; no Rust toolchain exists in the
// build image, so this header plays the role of the safe wrapper crate: same names, argument
// meaning and error behaviour (every failure becomes a turq::Error, nothing aborts).
//
//   candle / tur item                                        here
//   GgmlDType (block_size, type_size)                        turq::GgmlDType, block_size(), type_size()
//   QTensor::new / quantize / shape / dtype / dequantize     turq::QTensor
//     (src/weights/gguf_varbuilder.rs:62-79, src/weights/mod.rs:150)
//   QMatMul::from_arc / forward                              turq::QMatMul
//     (src/models/layers/linear.rs:24,69)
//   LinearX::Quantized { qmatmul, bias } / linear()          turq::LinearX
//     (src/models/layers/linear.rs:9-32, 50-70)
//
//   Qwen3MLP::forward (src/models/qwen3.rs:160-166)          turq::swiglu
//   ln -> projections (src/models/qwen3.rs:633-638)          turq::rmsnorm_forward_multi
//   lm_head -> LogitsProcessor::sample                       turq::QMatMul::lm_head_topk
//     (src/backend/engine.rs:528-529, 810-824)
//
// Header-only; link with libturq.so. Device pointers are the caller's (any allocator).
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "turq.h"

namespace turq {

struct Error : std::runtime_error {
  int32_t status;
  Error(int32_t st, const std::string& msg)
      : std::runtime_error(std::string(turq_status_string(st)) + ": " + msg), status(st) {}
};

enum class GgmlDType : int32_t { F32 = 0, F16 = 1, Q8_0 = 8, Q4K = 12, Q5K = 13, Q6K = 14, Q8K = 15, BF16 = 30 };
inline int block_size(GgmlDType t) { return turq_block_elems(static_cast<int32_t>(t)); }
inline int type_size(GgmlDType t) { return turq_block_bytes(static_cast<int32_t>(t)); }

enum class Mode : int32_t { Auto = 0, Int8Act = 1, ExactF32 = 2, TensorCore = 3 };

// One device + the scratch of the calls made through it (one thread / stream at a time).
class Context {
 public:
  explicit Context(int device = 0) {
    int32_t st = turq_ctx_create(device, &h_);
    if (st != TURQ_OK) throw Error(st, "turq_ctx_create");
  }
  ~Context() {
    if (h_) turq_ctx_destroy(h_);
  }
  Context(const Context&) = delete;
  Context& operator=(const Context&) = delete;
  turq_ctx* handle() const { return h_; }
  void check(int32_t st) const {
    if (st != TURQ_OK) throw Error(st, turq_last_error(h_));
  }
  // Synchronizes `stream` and throws if a kernel gave up a bounded device-side wait.
  void poll_status(void* stream = nullptr) const { check(turq_ctx_poll_status(h_, stream)); }
  // Sizes the scratch for the largest call so that no later call allocates.
  void reserve(int64_t max_m, int64_t max_k, int64_t max_n) const { check(turq_ctx_reserve(h_, max_m, max_k, max_n)); }
  // Pins what Mode::Auto means to one scheme for every row count (batch-independent results).
  void set_auto_policy(int32_t mode) const { check(turq_ctx_set_auto_policy(h_, mode)); }

 private:
  turq_ctx* h_ = nullptr;
};

// Immutable quantized weight [rows, cols] on the context's device (candle: QTensor).
class QTensor {
 public:
  // From GGUF wire-format blocks in host memory (what Content::tensor reads from the file).
  static std::shared_ptr<QTensor> from_host(std::shared_ptr<Context> ctx, GgmlDType dtype, int64_t rows, int64_t cols,
                                            const void* blocks, size_t nbytes) {
    turq_qtensor* h = nullptr;
    ctx->check(turq_qtensor_from_host(ctx->handle(), static_cast<int32_t>(dtype), rows, cols, blocks, nbytes, &h));
    return std::shared_ptr<QTensor>(new QTensor(std::move(ctx), h));
  }
  // candle: QTensor::quantize. dev_x is [rows, cols] f32 on the device; dev_blocks is the caller's
  // scratch of turq_row_bytes(dtype, cols) * rows bytes that receives the wire blocks on the way.
  static std::shared_ptr<QTensor> quantize(std::shared_ptr<Context> ctx, GgmlDType dtype, int64_t rows, int64_t cols,
                                           const float* dev_x, void* dev_blocks, void* stream = nullptr) {
    const int32_t dt = static_cast<int32_t>(dtype);
    ctx->check(turq_quantize_weights(ctx->handle(), dt, dev_x, rows, cols, dev_blocks, stream));
    turq_qtensor* h = nullptr;
    ctx->check(turq_qtensor_from_device(ctx->handle(), dt, rows, cols, dev_blocks, turq_row_bytes(dt, cols) * (size_t)rows, stream, &h));
    return std::shared_ptr<QTensor>(new QTensor(std::move(ctx), h));
  }
  ~QTensor() {
    if (h_) turq_qtensor_free(h_);
  }
  QTensor(const QTensor&) = delete;
  QTensor& operator=(const QTensor&) = delete;

  GgmlDType dtype() const { return dtype_; }
  std::pair<int64_t, int64_t> shape() const { return {rows_, cols_}; }
  size_t storage_size_in_bytes() const { return nbytes_; }
  // QTensor::dequantize: dev_out is [rows, cols] of out_dtype (F32 bit-exact, F16, BF16).
  void dequantize(void* dev_out, GgmlDType out_dtype = GgmlDType::F32, void* stream = nullptr) const {
    ctx_->check(turq_dequantize(ctx_->handle(), h_, static_cast<int32_t>(out_dtype), dev_out, stream));
  }
  // Embedding lookup on the quantized table: dev_out[i, :] = dequantize(row dev_ids[i]).
  void embedding(const int32_t* dev_ids, int64_t n_ids, void* dev_out, GgmlDType out_dtype = GgmlDType::F32,
                 void* stream = nullptr) const {
    ctx_->check(turq_embedding(ctx_->handle(), h_, dev_ids, n_ids, static_cast<int32_t>(out_dtype), dev_out, stream));
  }
  // Tensor-parallel shards (own memory).
  std::shared_ptr<QTensor> slice_rows(int64_t row0, int64_t n) const {
    turq_qtensor* h = nullptr;
    ctx_->check(turq_qtensor_slice_rows(ctx_->handle(), h_, row0, n, &h));
    return std::shared_ptr<QTensor>(new QTensor(ctx_, h));
  }
  std::shared_ptr<QTensor> slice_cols(int64_t col0, int64_t n) const {
    turq_qtensor* h = nullptr;
    ctx_->check(turq_qtensor_slice_cols(ctx_->handle(), h_, col0, n, &h));
    return std::shared_ptr<QTensor>(new QTensor(ctx_, h));
  }
  const turq_qtensor* handle() const { return h_; }
  const std::shared_ptr<Context>& context() const { return ctx_; }

 private:
  QTensor(std::shared_ptr<Context> ctx, turq_qtensor* h) : ctx_(std::move(ctx)), h_(h) {
    int32_t dt = 0;
    ctx_->check(turq_qtensor_info(h_, &dt, &rows_, &cols_, &nbytes_));
    dtype_ = static_cast<GgmlDType>(dt);
  }
  std::shared_ptr<Context> ctx_;
  turq_qtensor* h_ = nullptr;
  GgmlDType dtype_ = GgmlDType::F32;
  int64_t rows_ = 0, cols_ = 0;
  size_t nbytes_ = 0;
};

// y = x . W^T for a quantized W (candle: QMatMul).
class QMatMul {
 public:
  static QMatMul from_arc(std::shared_ptr<QTensor> w) { return QMatMul(std::move(w)); }
  // Device activations: x [m, cols] (F32 or BF16), y [m, rows] f32, stream-ordered.
  void forward(const void* dev_x, GgmlDType x_dtype, int64_t m, float* dev_y, const float* dev_bias = nullptr,
               Mode mode = Mode::Auto, void* stream = nullptr) const {
    const auto& c = w_->context();
    c->check(turq_qmatmul(c->handle(), w_->handle(), dev_x, static_cast<int32_t>(x_dtype), m, dev_y,
                          static_cast<int32_t>(mode), dev_bias, stream));
  }
  // Host activations, as tur holds them today (Device::Cpu): copies in, runs, copies out, syncs.
  std::vector<float> forward_host(const float* x, int64_t m, const float* bias = nullptr, Mode mode = Mode::Auto) const {
    const auto& c = w_->context();
    std::vector<float> y(static_cast<size_t>(m) * static_cast<size_t>(w_->shape().first));
    c->check(turq_qmatmul_host(c->handle(), w_->handle(), x, m, y.data(), static_cast<int32_t>(mode), bias));
    return y;
  }
  // Several linears that read the same x (attn_q|k|v, ffn_gate|up) in one call; ys[i] is [m, rows of mms[i]].
  static void forward_multi(const std::vector<const QMatMul*>& mms, const void* dev_x, GgmlDType x_dtype, int64_t m,
                            const std::vector<float*>& dev_ys, Mode mode = Mode::Auto, void* stream = nullptr) {
    if (mms.empty() || mms.size() != dev_ys.size()) throw Error(TURQ_E_INVALID_ARG, "forward_multi: weights and outputs must pair up");
    std::vector<const turq_qtensor*> qts;
    for (const QMatMul* mm : mms) qts.push_back(mm->w_->handle());
    const auto& c = mms[0]->w_->context();
    c->check(turq_qmatmul_multi(c->handle(), static_cast<int32_t>(qts.size()), qts.data(), dev_x, static_cast<int32_t>(x_dtype), m,
                                dev_ys.data(), static_cast<int32_t>(mode), nullptr, stream));
  }
  // The k best (logit, token id) pairs per row of x . W^T, best first, ties to the lower id.
  void lm_head_topk(const void* dev_x, GgmlDType x_dtype, int64_t m, int32_t k, float* dev_vals, int32_t* dev_ids,
                    int32_t id_offset = 0, float* dev_logits = nullptr, Mode mode = Mode::Auto, void* stream = nullptr) const {
    const auto& c = w_->context();
    c->check(turq_lm_head_topk(c->handle(), w_->handle(), dev_x, static_cast<int32_t>(x_dtype), m, k, id_offset, dev_vals, dev_ids,
                               dev_logits, static_cast<int32_t>(mode), stream));
  }
  const std::shared_ptr<QTensor>& weight() const { return w_; }

 private:
  explicit QMatMul(std::shared_ptr<QTensor> w) : w_(std::move(w)) {}
  std::shared_ptr<QTensor> w_;
};

// silu(x . Wg^T) * (x . Wu^T): one launch in the integer scheme.
inline void swiglu(const QMatMul& gate, const QMatMul& up, const void* dev_x, GgmlDType x_dtype, int64_t m, float* dev_out,
                   Mode mode = Mode::Auto, void* stream = nullptr) {
  const auto& c = gate.weight()->context();
  c->check(turq_qmatmul_swiglu(c->handle(), gate.weight()->handle(), up.weight()->handle(), dev_x, static_cast<int32_t>(x_dtype), m,
                               dev_out, static_cast<int32_t>(mode), stream));
}

// y_i = rmsnorm(x; weight, eps) . W_i^T; dev_h_out (nullable) receives the normalised rows.
inline void rmsnorm_forward_multi(const std::vector<const QMatMul*>& mms, const void* dev_x, GgmlDType x_dtype, int64_t m,
                                  const float* dev_norm_weight, float eps, float* dev_h_out, const std::vector<float*>& dev_ys,
                                  Mode mode = Mode::Auto, void* stream = nullptr) {
  if (mms.empty() || mms.size() != dev_ys.size()) throw Error(TURQ_E_INVALID_ARG, "rmsnorm_forward_multi: weights and outputs must pair up");
  std::vector<const turq_qtensor*> qts;
  for (const QMatMul* mm : mms) qts.push_back(mm->weight()->handle());
  const auto& c = mms[0]->weight()->context();
  c->check(turq_rmsnorm_qmatmul_multi(c->handle(), static_cast<int32_t>(qts.size()), qts.data(), dev_x, static_cast<int32_t>(x_dtype), m,
                                      dev_norm_weight, eps, dev_h_out, dev_ys.data(), static_cast<int32_t>(mode), nullptr, stream));
}

// The `Quantized` arm of tur's LinearX: QMatMul plus an optional f32 bias in device memory
// (the add is fused into the matmul epilogue).
class LinearX {
 public:
  LinearX(QMatMul mm, const float* dev_bias = nullptr) : mm_(std::move(mm)), dev_bias_(dev_bias) {}
  void forward(const void* dev_x, GgmlDType x_dtype, int64_t m, float* dev_y, void* stream = nullptr) const {
    mm_.forward(dev_x, x_dtype, m, dev_y, dev_bias_, Mode::Auto, stream);
  }

 private:
  QMatMul mm_;
  const float* dev_bias_;
};

}  // namespace turq
