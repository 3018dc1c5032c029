// Host-side mirror of the reference's tensor interface for the training hot path, in C++ over the
// C ABI of libheirloom_b200 (the reference is Rust; this is the layer a maintainer would bind in its
// place).  What is mirrored, with the same names, argument meaning and error behaviour:
//   * Tensor handle and storage (src/tensor.rs:39-58, src/storage.rs:29-41): shared handle with id,
//     storage, shape, element strides, storage offset, dtype, device, requires_grad, grad, grad_fn;
//   * metadata-only views view / reshape / transpose / permute / narrow / expand
//     (src/tensor.rs:2429-2688);
//   * the operator catalog, 18 schemas (src/dispatch.rs:6-25, :93-238);
//   * custom unary ops and their registry (src/extension.rs:4-155, src/tensor.rs:4496-4519);
//   * the ops of the training step, each routed to the device kernels first, as the reference's
//     `cuda_*` early returns do (tests/cuda_dispatch_guards.rs:4-76);
//   * the autograd driver: depth-first topological order, reverse walk, accumulation by tensor
//     identity, leaf gradients kept, graph released (src/tensor.rs:1854-1942,
//     src/tensor/autograd.rs:2922-2943);
//   * Linear, LayerNorm, Embedding, Gelu, CausalSelfAttention, FeedForward, TransformerBlock and
//     AdamW (src/nn.rs).
// Compute runs on the GPU only: an op on a host tensor reports an error instead of falling back
// to host arithmetic.  Host tensors exist as containers (construction, views, upload, download)
// and for custom unary ops, whose callbacks are host functions by definition.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace heirloom {

enum class DType { F32, F64, I64, Bool, BF16 };
inline bool is_floating(DType d) { return d == DType::F32 || d == DType::F64 || d == DType::BF16; }
const char* dtype_name(DType d);

struct Device {
  enum Kind { Cpu, Cuda } kind = Cpu;
  int ordinal = 0;
  static Device cpu() { return Device{Cpu, 0}; }
  static Device cuda(int ordinal) { return Device{Cuda, ordinal}; }
  bool operator==(const Device& o) const { return kind == o.kind && (kind == Cpu || ordinal == o.ordinal); }
  bool operator!=(const Device& o) const { return !(*this == o); }
};

// TensorError (src/lib.rs): the kind is part of the message prefix, as in the reference's Display.
class TensorError : public std::runtime_error {
 public:
  enum Kind { InvalidOperation, Shape, DeviceError, Autograd };
  TensorError(Kind kind, const std::string& message);
  Kind kind() const { return kind_; }
 private:
  Kind kind_;
};

// ---- operator catalog (src/dispatch.rs:6-92) ----------------------------------------------------------
enum class Operator {
  Add, Sub, Mul, Div, Matmul, Relu, Gelu, SoftmaxDim, CrossEntropyForLogits, Sum, Mean, SumDim, MeanDim,
  LayerNormLastDim, Embedding, MaskedFill, ArgmaxLastDim, CausalSelfAttention
};
enum class OperatorKind {
  Binary, Unary, MatrixMultiply, Loss, ReductionAll, ReductionDim, Normalization, Indexing, Masking, Selection, Attention
};
enum class DTypeRule {
  ArithmeticPromotion, FloatingPromotion, PreserveFloating, SumReduction, MeanReduction, EmbeddingLookup, MaskPreserve,
  ArgmaxIndex, SameFloatingInputs
};
enum class AliasPolicy { FreshOutput };
enum class AutogradPolicy { FloatingInputs, NonDifferentiable };
struct OperatorInfo {
  Operator op;
  const char* name;
  OperatorKind kind;
  DTypeRule dtype_rule;
  AliasPolicy alias_policy;
  AutogradPolicy autograd_policy;
  bool returns_fresh_output() const { return alias_policy == AliasPolicy::FreshOutput; }
  bool should_record_autograd(DType output_dtype, bool input_requires_grad) const {
    return autograd_policy == AutogradPolicy::FloatingInputs && input_requires_grad && is_floating(output_dtype);
  }
};
const std::vector<OperatorInfo>& operator_catalog();
const OperatorInfo& operator_schema(Operator op);

// ---- custom unary ops (src/extension.rs) --------------------------------------------------------------
struct CustomUnaryForwardContext {
  const char* name;
  const std::vector<double>& input;
  const std::vector<size_t>& shape;
  DType dtype;
  Device device;
};
struct CustomUnaryBackwardContext {
  const char* name;
  const std::vector<double>& input;
  const std::vector<double>& output;
  const std::vector<double>& grad_output;
  const std::vector<size_t>& shape;
  DType dtype;
  Device device;
};
using CustomUnaryForward = std::vector<double> (*)(const CustomUnaryForwardContext&);
using CustomUnaryBackward = std::vector<double> (*)(const CustomUnaryBackwardContext&);
class CustomUnaryOp {
 public:
  // Names: non-empty, at most 128 bytes, characters [A-Za-z0-9_.:-] (src/extension.rs:157-178).
  CustomUnaryOp(const char* name, CustomUnaryForward forward, CustomUnaryBackward backward);
  const char* name() const { return name_; }
  CustomUnaryForward forward_fn() const { return forward_; }
  CustomUnaryBackward backward_fn() const { return backward_; }
 private:
  const char* name_;
  CustomUnaryForward forward_;
  CustomUnaryBackward backward_;
};
class CustomUnaryRegistry {
 public:
  void register_op(const CustomUnaryOp& op);  // a second op of the same name is an InvalidOperation
  std::optional<CustomUnaryOp> get(const std::string& name) const;
  const std::vector<CustomUnaryOp>& operators() const { return ops_; }
  size_t len() const { return ops_.size(); }
  bool is_empty() const { return ops_.empty(); }
 private:
  std::vector<CustomUnaryOp> ops_;
};

// ---- tensor -----------------------------------------------------------------------------------------
struct Storage;      // host vector or device buffer, with a version counter
struct TensorInner;
struct GradFn;

class Tensor {
 public:
  Tensor() = default;
  // constructors (host tensors, row-major contiguous)
  static Tensor from_vec(const std::vector<float>& data, const std::vector<size_t>& shape, bool requires_grad = false);
  static Tensor from_f64(const std::vector<double>& data, const std::vector<size_t>& shape, bool requires_grad = false);
  static Tensor from_i64(const std::vector<int64_t>& data, const std::vector<size_t>& shape);
  static Tensor zeros(const std::vector<size_t>& shape, DType dtype = DType::F32, Device device = Device::cpu());

  bool defined() const { return static_cast<bool>(inner_); }
  uint64_t id() const;
  const std::vector<size_t>& shape() const;
  const std::vector<size_t>& strides() const;  // in elements
  size_t storage_offset() const;
  DType dtype() const;
  Device device() const;
  size_t numel() const;
  size_t ndim() const { return shape().size(); }
  bool is_contiguous() const;
  bool shares_storage_with(const Tensor& other) const;
  size_t storage_version() const;

  bool requires_grad() const;
  Tensor& set_requires_grad(bool on);  // leaves only
  bool is_leaf() const;
  std::optional<Tensor> grad() const;
  std::vector<double> grad_f64() const;  // error when there is no gradient
  void zero_grad();

  // values in logical (row-major over the shape) order; a device tensor is copied to the host after
  // the compute stream has drained
  std::vector<double> data_f64() const;
  std::vector<float> data_f32() const;
  std::vector<int64_t> data_i64() const;
  double item() const;  // one-element tensors

  Tensor to_device(Device device) const;  // f32 and i64 tensors; detached copy that keeps requires_grad
  Tensor cuda(int ordinal = 0) const { return to_device(Device::cuda(ordinal)); }
  Tensor cpu() const { return to_device(Device::cpu()); }
  Tensor detach() const;

  // views: metadata only, each recorded for autograd
  Tensor view(const std::vector<size_t>& shape) const;     // contiguous tensors only
  Tensor reshape(const std::vector<size_t>& shape) const;  // a view when contiguous; host tensors are copied otherwise
  Tensor transpose(size_t dim0, size_t dim1) const;
  Tensor permute(const std::vector<size_t>& dims) const;
  Tensor narrow(size_t dim, size_t start, size_t length) const;
  Tensor expand(const std::vector<size_t>& shape) const;

  // ops of the hot path
  Tensor add(const Tensor& other) const;  // same shape, or [rows, cols] + [cols]
  Tensor sub(const Tensor& other) const;
  Tensor mul(const Tensor& other) const;
  Tensor div(const Tensor& other) const;
  Tensor matmul(const Tensor& other) const;  // rank-2 operands, any element strides
  Tensor relu() const;
  Tensor gelu() const;
  Tensor softmax_dim(size_t dim) const;  // rank 2, last dimension
  Tensor sum() const;
  Tensor mean() const;
  Tensor layer_norm_last_dim(const Tensor& weight, const Tensor& bias, double eps = 1e-5) const;
  static Tensor embedding(const Tensor& weight, const Tensor& indices);
  static Tensor causal_self_attention(const Tensor& q, const Tensor& k, const Tensor& v, size_t n_heads);
  Tensor cross_entropy_for_logits(const Tensor& targets) const;  // [rows, classes] logits, i64 targets
  Tensor apply_custom_unary(const CustomUnaryOp& op) const;

  void backward() const;  // one-element tensors; seeds the gradient with 1

  // used by the optimizer and by tests
  std::shared_ptr<TensorInner> inner() const { return inner_; }
  explicit Tensor(std::shared_ptr<TensorInner> inner) : inner_(std::move(inner)) {}

 private:
  std::shared_ptr<TensorInner> inner_;
};

// Scope in which ops record no autograd graph (src/autograd mode `no_grad`).
class NoGradGuard {
 public:
  NoGradGuard();
  ~NoGradGuard();
 private:
  bool previous_;
};
template <typename F>
auto no_grad(F&& f) -> decltype(f()) {
  NoGradGuard guard;
  return f();
}
bool grad_enabled();

// Counters of the device library for the context of `ordinal` (launches, allocations).
struct RuntimeCounters { unsigned long long launches = 0, allocations = 0; };
RuntimeCounters cuda_runtime_counters(int ordinal = 0);
void synchronize(int ordinal = 0);

// ---- modules (src/nn.rs) ----------------------------------------------------------------------------
namespace nn {

struct Linear {  // y = x·Wᵀ + b, W [out, in] (src/nn.rs:454-475)
  Tensor weight, bias;
  Linear() = default;
  Linear(const Tensor& weight, const Tensor& bias) : weight(weight), bias(bias) {}
  Tensor forward(const Tensor& x) const;  // x [rows, in]
  std::vector<Tensor> parameters() const { return {weight, bias}; }
};
struct LayerNorm {  // src/nn.rs:650-653
  Tensor weight, bias;
  double eps = 1e-5;
  Tensor forward(const Tensor& x) const { return x.layer_norm_last_dim(weight, bias, eps); }
  std::vector<Tensor> parameters() const { return {weight, bias}; }
};
struct Embedding {  // src/nn.rs:597-609
  Tensor weight;
  Tensor forward(const Tensor& indices) const { return Tensor::embedding(weight, indices); }
  std::vector<Tensor> parameters() const { return {weight}; }
};
struct Gelu {  // src/nn.rs:534-546
  Tensor forward(const Tensor& x) const { return x.gelu(); }
};
struct CausalSelfAttention {  // q, k, v, out projections around the fused attention op (src/nn.rs:807-814)
  Linear q_proj, k_proj, v_proj, out_proj;
  size_t n_heads = 1;
  Tensor forward(const Tensor& x, size_t batch, size_t time) const;  // x [batch*time, d]
  std::vector<Tensor> parameters() const;
};
struct FeedForward {  // fc1 -> gelu -> fc2 (src/nn.rs:888-891)
  Linear fc1, fc2;
  Tensor forward(const Tensor& x) const { return fc2.forward(fc1.forward(x).gelu()); }
  std::vector<Tensor> parameters() const;
};
struct TransformerBlock {  // pre-LN: r = x + attn(ln1 x); y = r + ff(ln2 r) (src/nn.rs:988-993)
  LayerNorm ln1, ln2;
  CausalSelfAttention attention;
  FeedForward feed_forward;
  Tensor forward(const Tensor& x, size_t batch, size_t time) const;
  std::vector<Tensor> parameters() const;
};

// Coupled-decay AdamW over device parameters (src/nn.rs:1941-2005, step_mut :2156-2220, CUDA body
// :2467-2505): parameters without a gradient are skipped; the step counter advances once per call.
class AdamW {
 public:
  AdamW(std::vector<Tensor> parameters, double lr = 1e-3, double beta1 = 0.9, double beta2 = 0.999, double eps = 1e-8,
        double weight_decay = 0.01, std::optional<double> clip_norm = std::nullopt);
  void zero_grad();
  void step();
  int step_count() const { return step_; }
 private:
  std::vector<Tensor> params_;
  std::vector<Tensor> m_, v_;
  double lr_, beta1_, beta2_, eps_, weight_decay_;
  std::optional<double> clip_norm_;
  int step_ = 0;
};

}  // namespace nn
}  // namespace heirloom
