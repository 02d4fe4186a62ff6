// Header-only C++ layer over the C ABI (vkllama_b200.h) that keeps vkllama's own class
// surface: namespace vkllama, GPUDevice, Tensor, Command, class Op and one class per
// operator with the constructor and operator() argument lists of src/ops/*.h, plus a
// Model with init-by-tensor-name and operator()(toks, offset) as models/llama2.h:322-854.
// abseil is not required: Status / StatusOr below are minimal stand-ins with the spelling
// the reference uses (ok(), status(), operator*, operator->, message(), ToString()).
#ifndef VKLLAMA_B200_CPP_H_
#define VKLLAMA_B200_CPP_H_

#include <array>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

extern "C" {
#include "../vkllama_b200.h"
}

namespace absl_shim {
enum class StatusCode : int { kOk = 0, kInvalidArgument = 3, kResourceExhausted = 8, kFailedPrecondition = 9, kOutOfRange = 11, kUnimplemented = 12, kInternal = 13 };
class Status {
 public:
  Status() = default;
  Status(StatusCode c, std::string m) : code_(c), msg_(std::move(m)) {}
  bool ok() const { return code_ == StatusCode::kOk; }
  StatusCode code() const { return code_; }
  const std::string &message() const { return msg_; }
  std::string ToString() const { return ok() ? "OK" : "[" + std::to_string((int)code_) + "] " + msg_; }

 private:
  StatusCode code_ = StatusCode::kOk;
  std::string msg_;
};
inline Status OkStatus() { return Status(); }
inline Status InvalidArgumentError(std::string m) { return Status(StatusCode::kInvalidArgument, std::move(m)); }
inline Status OutOfRangeError(std::string m) { return Status(StatusCode::kOutOfRange, std::move(m)); }
inline Status InternalError(std::string m) { return Status(StatusCode::kInternal, std::move(m)); }
inline Status UnimplementedError(std::string m) { return Status(StatusCode::kUnimplemented, std::move(m)); }
template <class T>
class StatusOr {
 public:
  StatusOr(const Status &s) : st_(s) {}
  StatusOr(T v) : val_(std::move(v)), has_(true) {}
  bool ok() const { return has_; }
  const Status &status() const { return st_; }
  T &operator*() { return val_; }
  const T &operator*() const { return val_; }
  T *operator->() { return &val_; }
  const T *operator->() const { return &val_; }

 private:
  Status st_;
  T val_{};
  bool has_ = false;
};
}  // namespace absl_shim

namespace vkllama {
namespace absl = ::absl_shim;

// src/core/common.h:15-22
typedef enum : int { FP32 = 0, FP16, UINT32, INT8, Q8_0 } DType;

#define VKLLAMA_STATUS_OK(__expr)              \
  if (auto __s = (__expr); !__s.ok()) {        \
    return __s;                                \
  }

inline absl::Status ToStatus(int code) {
  return code == VKL_OK ? absl::OkStatus() : absl::Status(static_cast<absl::StatusCode>(code), vkl_last_error());
}

// src/core/gpu_device.h:13-62
class GPUDevice {
 public:
  explicit GPUDevice(int dev = 0) : ordinal_(dev) {}
  ~GPUDevice() { vkl_device_destroy(h_); }
  GPUDevice(const GPUDevice &) = delete;
  absl::Status init() { return ToStatus(vkl_device_create(ordinal_, &h_)); }
  size_t subgroup_size() const { return 32; }
  bool support_16bit_storage() const { return true; }
  bool support_fp16_arithmetic() const { return true; }
  vkl_device *handle() const { return h_; }

 private:
  int ordinal_;
  vkl_device *h_ = nullptr;
};

// src/core/tensor.h:16-90: a value-type handle, copies share the buffer.
class Tensor {
 public:
  using DType = ::vkllama::DType;
  Tensor() = default;
  Tensor(int c, int h, int w, GPUDevice *dev, DType dtype = FP32, bool /*visable*/ = false) : dev_(dev) {
    if (dev && dev->handle()) vkl_tensor_create(dev->handle(), c, h, w, dtype, &t_);
  }
  Tensor(const Tensor &o) : dev_(o.dev_), t_(o.t_) {
    if (t_) vkl_tensor_retain(t_);
  }
  Tensor(Tensor &&o) noexcept : dev_(o.dev_), t_(o.t_) { o.t_ = nullptr; }
  Tensor &operator=(Tensor o) {
    std::swap(dev_, o.dev_);
    std::swap(t_, o.t_);
    return *this;
  }
  ~Tensor() { vkl_tensor_release(t_); }
  static Tensor like(const Tensor &o) { return Tensor((int)o.channels(), (int)o.height(), (int)o.width(), o.dev_, o.dtype()); }
  static Tensor Borrow(vkl_tensor *t, GPUDevice *dev) {  // an op-owned output: retain it
    Tensor r;
    r.dev_ = dev;
    r.t_ = t;
    if (t) vkl_tensor_retain(t);
    return r;
  }
  absl::Status create() { return t_ ? absl::OkStatus() : absl::InternalError("tensor allocation failed: " + std::string(vkl_last_error())); }
  size_t channels() const { return shape6()[0]; }
  size_t height() const { return shape6()[1]; }
  size_t width() const { return shape6()[2]; }
  size_t cs() const { return shape6()[3]; }
  size_t hs() const { return shape6()[4]; }
  size_t ws() const { return shape6()[5]; }
  std::array<size_t, 3> shape() const { return {channels(), height(), width()}; }
  size_t size() const { return t_ ? channels() * height() * width() : 0; }
  size_t bytes() const {
    size_t b = 0;
    if (t_) vkl_tensor_bytes(t_, &b);
    return b;
  }
  DType dtype() const {
    int d = FP32;
    if (t_) vkl_tensor_dtype(t_, &d);
    return (DType)d;
  }
  absl::Status reshape(size_t c, size_t h, size_t w) { return ToStatus(vkl_tensor_reshape(t_, c, h, w)); }
  Tensor view(size_t c, size_t h, size_t w) {
    vkl_tensor *v = nullptr;
    vkl_tensor_view(t_, c, h, w, &v);
    Tensor r;
    r.dev_ = dev_;
    r.t_ = v;
    return r;
  }
  vkl_tensor *handle() const { return t_; }

 private:
  std::array<uint32_t, 6> shape6() const {
    std::array<uint32_t, 6> s{};
    if (t_) vkl_tensor_shape(t_, s.data());
    return s;
  }
  GPUDevice *dev_ = nullptr;
  vkl_tensor *t_ = nullptr;
};

// src/core/command.h:26-483
class Command {
 public:
  explicit Command(GPUDevice *dev) : dev_(dev) {}
  ~Command() { vkl_command_destroy(h_); }
  Command(const Command &) = delete;
  absl::Status init() { return ToStatus(vkl_command_create(dev_->handle(), &h_)); }
  absl::Status begin() { return ToStatus(vkl_command_begin(h_)); }
  absl::Status end() { return ToStatus(vkl_command_end(h_)); }
  absl::Status submit() { return ToStatus(vkl_command_submit(h_)); }
  absl::Status wait() { return ToStatus(vkl_command_wait(h_)); }
  absl::Status submit_and_wait() { return ToStatus(vkl_command_submit_and_wait(h_)); }
  template <typename T>
  absl::Status upload(T const *from, size_t n, Tensor &to) {
    return ToStatus(vkl_command_upload(h_, from, n * sizeof(T), to.handle()));
  }
  template <typename T>
  absl::Status download(Tensor &from, T *to, size_t n) {
    return ToStatus(vkl_command_download(h_, from.handle(), to, n * sizeof(T)));
  }
  vkl_command *handle() const { return h_; }

 private:
  GPUDevice *dev_;
  vkl_command *h_ = nullptr;
};

// src/ops/op.h:14-25
class Op {
 public:
  Op(GPUDevice *dev, Command *command) noexcept : dev_(dev), command_(command) {}
  virtual absl::Status init() noexcept { return op_ ? ToStatus(vkl_op_init(op_)) : absl::InternalError(vkl_last_error()); }
  virtual uint64_t time() noexcept {
    uint64_t us = 0;
    if (op_) vkl_op_time(op_, &us);
    return us;
  }
  virtual ~Op() { vkl_op_destroy(op_); }
  Op(const Op &) = delete;

 protected:
  absl::StatusOr<Tensor> out(int status, vkl_tensor *t) {
    if (status != VKL_OK) return ToStatus(status);
    return Tensor::Borrow(t, dev_);
  }
  GPUDevice *dev_;
  Command *command_;
  vkl_op *op_ = nullptr;
};

// src/ops/mat_mul.h:12-27
class MatMul : public Op {
 public:
  MatMul(GPUDevice *dev, Command *command, Tensor weight, const float scale = 1.0f, const float bias = .0f, const int act = 0,
         const int broadcast_type = 0, const bool transpose_b = false, const Tensor::DType a_dtype = FP16, const Tensor::DType b_dtype = FP16)
      : Op(dev, command), weight_(weight) {
    vkl_matmul_create(dev->handle(), command->handle(), weight_.handle(), scale, bias, act, broadcast_type, transpose_b, a_dtype, b_dtype, &op_);
  }
  MatMul(GPUDevice *dev, Command *command, const float scale = 1.0f, const float bias = .0f, const int act = 0, const int broadcast_type = 0,
         const bool transpose_b = false, const Tensor::DType a_dtype = FP16, const Tensor::DType b_dtype = FP16)
      : Op(dev, command) {
    vkl_matmul_create(dev->handle(), command->handle(), nullptr, scale, bias, act, broadcast_type, transpose_b, a_dtype, b_dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor a) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_matmul_run(op_, a.handle(), nullptr, &o);  // sequenced before `o` is read
    return out(st, o);
  }
  absl::StatusOr<Tensor> operator()(Tensor a, Tensor b) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_matmul_run(op_, a.handle(), b.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }

 private:
  Tensor weight_;
};

// src/ops/feed_forward.h:17-22 (w1 = gate, w2 = down, w3 = up)
class FeedForward : public Op {
 public:
  FeedForward(GPUDevice *dev, Command *command, Tensor w1, Tensor w2, Tensor w3, const bool transposed_weight = false,
              const Tensor::DType dtype = FP16)
      : Op(dev, command), w1_(w1), w2_(w2), w3_(w3) {
    vkl_feed_forward_create(dev->handle(), command->handle(), w1_.handle(), w2_.handle(), w3_.handle(), transposed_weight, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor X) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_feed_forward_run(op_, X.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }

 private:
  Tensor w1_, w2_, w3_;
};

// src/ops/multiheadattention_v2.h:25-35
class MultiHeadAttentionV2 : public Op {
 public:
  MultiHeadAttentionV2(GPUDevice *dev, Command *command, Tensor wk, Tensor wq, Tensor wv, Tensor wo, const int maxlen, const int dim,
                       const bool transposed_weight = false, Tensor::DType dtype = FP16, const bool use_kvcache = false,
                       const bool clip_output = false)
      : Op(dev, command), wk_(wk), wq_(wq), wv_(wv), wo_(wo) {
    vkl_mha_create(dev->handle(), command->handle(), wk_.handle(), wq_.handle(), wv_.handle(), wo_.handle(), maxlen, dim, transposed_weight,
                   dtype, use_kvcache, clip_output, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor X, const size_t offset = 0) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_mha_run(op_, X.handle(), offset, &o);  // sequenced before `o` is read
    return out(st, o);
  }

 private:
  Tensor wk_, wq_, wv_, wo_;
};

// src/ops/update_kv_cache.h:13-18
class UpdateKVCache : public Op {
 public:
  UpdateKVCache(GPUDevice *dev, Command *command, const Tensor::DType dtype) : Op(dev, command) {
    vkl_update_kvcache_create(dev->handle(), command->handle(), dtype, &op_);
  }
  absl::Status operator()(Tensor cache, Tensor key_or_value, const uint32_t offset) noexcept {
    return ToStatus(vkl_update_kvcache_run(op_, cache.handle(), key_or_value.handle(), offset));
  }
};

// src/ops/rms_norm.h:12-16
class RMSNorm : public Op {
 public:
  RMSNorm(GPUDevice *dev, Command *command, Tensor weight, const float eps = 1e-3f, const Tensor::DType dtype = FP16)
      : Op(dev, command), weight_(weight) {
    vkl_rms_norm_create(dev->handle(), command->handle(), weight_.handle(), eps, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor x) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_rms_norm_run(op_, x.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }

 private:
  Tensor weight_;
};

// src/ops/rope.h:15-21
class Rope : public Op {
 public:
  Rope(GPUDevice *dev, Command *command, const int maxlen, const int dim, const Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_rope_create(dev->handle(), command->handle(), maxlen, dim, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor query, const size_t offset = 0) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_rope_run(op_, query.handle(), offset, &o);  // sequenced before `o` is read
    return out(st, o);
  }
};

// src/ops/softmax.h:14-18
class Softmax : public Op {
 public:
  Softmax(GPUDevice *dev, Command *command, bool seq_mask = false, const float temp = 1.0f, const Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_softmax_create(dev->handle(), command->handle(), seq_mask, temp, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor a, size_t offset = 0) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_softmax_run(op_, a.handle(), offset, &o);  // sequenced before `o` is read
    return out(st, o);
  }
};

// src/ops/argop.h:13-156
template <int op_type>
class ArgOp : public Op {
 public:
  ArgOp(GPUDevice *dev, Command *command, const Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_argop_create(dev->handle(), command->handle(), op_type, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor in) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_argop_run(op_, in.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }
};
using ArgMax = ArgOp<0>;
using ArgMin = ArgOp<1>;

// src/ops/embedding.h:13-18
class Embedding : public Op {
 public:
  Embedding(GPUDevice *dev, Command *command, Tensor vocab, const uint32_t UNK, const Tensor::DType dtype = FP16) : Op(dev, command), vocab_(vocab) {
    vkl_embedding_create(dev->handle(), command->handle(), vocab_.handle(), UNK, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor indices) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_embedding_run(op_, indices.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }

 private:
  Tensor vocab_;
};

// src/ops/elementwise.h:16-21
class ElementWise : public Op {
 public:
  ElementWise(GPUDevice *dev, Command *command, const int type, Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_elementwise_create(dev->handle(), command->handle(), type, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor x, Tensor y) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_elementwise_run(op_, x.handle(), y.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }
  absl::StatusOr<Tensor> operator()(Tensor x, float y) noexcept {  // elementwise.cpp:104-133: in place in x
    vkl_tensor *o = nullptr;
    const int st = vkl_elementwise_run_scalar(op_, x.handle(), y, &o);
    return out(st, o);
  }
};

// src/ops/concat.h:10-17
class Concat : public Op {
 public:
  Concat(GPUDevice *dev, Command *command, const int num, const int axis, Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_concat_create(dev->handle(), command->handle(), num, axis, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(const std::vector<Tensor> &inputs) noexcept {
    std::vector<vkl_tensor *> hs;
    for (const Tensor &t : inputs) hs.push_back(t.handle());
    vkl_tensor *o = nullptr;
    const int st = vkl_concat_run(op_, hs.data(), hs.size(), &o);
    return out(st, o);
  }
};

// src/ops/reduce.h:18-67: 0 sum, 1 max, 2 min, 3 mean
class Reduce : public Op {
 public:
  Reduce(GPUDevice *dev, Command *command, int op_type, Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_reduce_create(dev->handle(), command->handle(), op_type, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor a) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_reduce_run(op_, a.handle(), &o);
    return out(st, o);
  }
};

// src/ops/read_kvcache_op.h:10-16
class ReadKVCache : public Op {
 public:
  ReadKVCache(GPUDevice *dev, Command *command) : Op(dev, command) { vkl_read_kvcache_create(dev->handle(), command->handle(), &op_); }
  absl::StatusOr<Tensor> operator()(Tensor cache, uint32_t offset, uint32_t len) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_read_kvcache_run(op_, cache.handle(), offset, len, &o);
    return out(st, o);
  }
};

// src/ops/transpose.h:14-19
class Transpose : public Op {
 public:
  Transpose(GPUDevice *dev, Command *command, const int type, Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_transpose_create(dev->handle(), command->handle(), type, dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor in) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_transpose_run(op_, in.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }
};

// src/ops/slice.h:13-18
class Slice : public Op {
 public:
  Slice(GPUDevice *dev, Command *command, Tensor::DType dtype = FP16) : Op(dev, command) {
    vkl_slice_create(dev->handle(), command->handle(), dtype, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor in, const std::array<uint32_t, 3> &starts, const std::array<uint32_t, 3> &extents) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_slice_run(op_, in.handle(), starts.data(), extents.data(), &o);  // sequenced before `o` is read
    return out(st, o);
  }
};

// src/ops/cast.h:15-20
class Cast : public Op {
 public:
  Cast(GPUDevice *dev, Command *command, const Tensor::DType from, const Tensor::DType to) : Op(dev, command) {
    vkl_cast_create(dev->handle(), command->handle(), from, to, &op_);
  }
  absl::StatusOr<Tensor> operator()(Tensor in) noexcept {
    vkl_tensor *o = nullptr;
    const int st = vkl_cast_run(op_, in.handle(), &o);  // sequenced before `o` is read
    return out(st, o);
  }
};

// models/llama2.h:322-854. The reference's init() takes gguflib maps; here the same
// information arrives as hyper-parameters plus one call per GGUF tensor (name, GGUF type
// id 0/1/8 = FP32/FP16/Q8_0 as at llama2.h:382-397, raw payload).
struct ModelConfig {
  uint32_t dim = 0, head_count = 0, ffn = 0, vocab = 0, block_count = 0, context_length = 0;
  float layer_norm_rms_epsilon = 1e-5f;
  DType weight_dtype = Q8_0;
};
class Model {
 public:
  explicit Model(int dev = 0) : dev_(dev) {}
  ~Model() {
    vkl_model_destroy(m_);
    delete gpu_;
  }
  Model(const Model &) = delete;
  absl::Status init(const ModelConfig &c) {
    gpu_ = new GPUDevice(dev_);
    VKLLAMA_STATUS_OK(gpu_->init());
    vkl_model_config k{};
    k.dim = c.dim; k.heads = c.head_count; k.ffn = c.ffn; k.vocab = c.vocab; k.layers = c.block_count; k.maxlen = c.context_length;
    k.eps = c.layer_norm_rms_epsilon;
    k.final_eps = 1e-6f;  // hard-coded for the output norm at llama2.h:268
    k.weight_dtype = c.weight_dtype;
    k.tp_rank = 0;
    k.tp_size = 1;
    vocab_ = c.vocab;
    return ToStatus(vkl_model_create(gpu_->handle(), &k, &m_));
  }
  absl::Status load_tensor(const std::string &name, uint32_t gguf_type, const void *weights_data, size_t bsize) {
    const int dt = gguf_type == 0 ? FP32 : gguf_type == 1 ? FP16 : gguf_type == 8 ? Q8_0 : INT8;
    return ToStatus(vkl_model_set_weight(m_, name.c_str(), dt, weights_data, bsize));
  }
  absl::StatusOr<std::vector<float>> operator()(std::vector<uint32_t> const &toks, const size_t offset) {
    std::vector<float> logits(vocab_);
    int s = vkl_model_forward(m_, toks.data(), toks.size(), offset, logits.data());
    if (s != VKL_OK) return ToStatus(s);
    return logits;
  }
  vkl_model *handle() const { return m_; }

 private:
  int dev_;
  GPUDevice *gpu_ = nullptr;
  vkl_model *m_ = nullptr;
  uint32_t vocab_ = 0;
};

}  // namespace vkllama
#endif  // VKLLAMA_B200_CPP_H_
