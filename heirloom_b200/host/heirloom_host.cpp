// Implementation of the host-side tensor interface over the C ABI of libheirloom_b200.
#include "heirloom.hpp"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <map>
#include <numeric>
#include <unordered_map>
#include <unordered_set>

#include "../../include/heirloom_b200.h"

namespace heirloom {

// ---- errors -------------------------------------------------------------------------------------------
static std::string prefix(TensorError::Kind k) {
  switch (k) {
    case TensorError::InvalidOperation: return "invalid operation: ";
    case TensorError::Shape: return "shape error: ";
    case TensorError::DeviceError: return "device error: ";
    default: return "autograd error: ";
  }
}
TensorError::TensorError(Kind kind, const std::string& message) : std::runtime_error(prefix(kind) + message), kind_(kind) {}
static void check(int rc) {
  if (rc != HL_OK) throw TensorError(TensorError::DeviceError, hl_last_error());  // CudaError -> TensorError::Device
}
const char* dtype_name(DType d) {
  switch (d) {
    case DType::F32: return "f32";
    case DType::F64: return "f64";
    case DType::I64: return "i64";
    case DType::Bool: return "bool";
    default: return "bf16";
  }
}

// ---- operator catalog ---------------------------------------------------------------------------------
const std::vector<OperatorInfo>& operator_catalog() {
  using O = Operator; using K = OperatorKind; using R = DTypeRule;
  const AliasPolicy F = AliasPolicy::FreshOutput;
  const AutogradPolicy G = AutogradPolicy::FloatingInputs;
  static const std::vector<OperatorInfo> catalog = {
      {O::Add, "aten.add", K::Binary, R::ArithmeticPromotion, F, G},
      {O::Sub, "aten.sub", K::Binary, R::ArithmeticPromotion, F, G},
      {O::Mul, "aten.mul", K::Binary, R::ArithmeticPromotion, F, G},
      {O::Div, "aten.div", K::Binary, R::ArithmeticPromotion, F, G},
      {O::Matmul, "aten.matmul", K::MatrixMultiply, R::FloatingPromotion, F, G},
      {O::Relu, "aten.relu", K::Unary, R::PreserveFloating, F, G},
      {O::Gelu, "aten.gelu", K::Unary, R::PreserveFloating, F, G},
      {O::SoftmaxDim, "aten.softmax.dim", K::Unary, R::PreserveFloating, F, G},
      {O::CrossEntropyForLogits, "heirloom.cross_entropy_for_logits", K::Loss, R::PreserveFloating, F, G},
      {O::Sum, "aten.sum", K::ReductionAll, R::SumReduction, F, G},
      {O::Mean, "aten.mean", K::ReductionAll, R::MeanReduction, F, G},
      {O::SumDim, "aten.sum.dim", K::ReductionDim, R::SumReduction, F, G},
      {O::MeanDim, "aten.mean.dim", K::ReductionDim, R::MeanReduction, F, G},
      {O::LayerNormLastDim, "aten.layer_norm.last_dim", K::Normalization, R::SameFloatingInputs, F, G},
      {O::Embedding, "aten.embedding", K::Indexing, R::EmbeddingLookup, F, G},
      {O::MaskedFill, "aten.masked_fill", K::Masking, R::MaskPreserve, F, G},
      {O::ArgmaxLastDim, "aten.argmax.last_dim", K::Selection, R::ArgmaxIndex, F, AutogradPolicy::NonDifferentiable},
      {O::CausalSelfAttention, "heirloom.causal_self_attention", K::Attention, R::SameFloatingInputs, F, G},
  };
  return catalog;
}
const OperatorInfo& operator_schema(Operator op) {
  for (const auto& s : operator_catalog())
    if (s.op == op) return s;
  throw TensorError(TensorError::InvalidOperation, "operator without a schema");
}

// ---- custom unary ops ---------------------------------------------------------------------------------
CustomUnaryOp::CustomUnaryOp(const char* name, CustomUnaryForward forward, CustomUnaryBackward backward)
    : name_(name), forward_(forward), backward_(backward) {
  const std::string n = name ? name : "";
  if (n.find_first_not_of(" \t\n\r") == std::string::npos)
    throw TensorError(TensorError::InvalidOperation, "custom op name cannot be empty");
  if (n.size() > 128)
    throw TensorError(TensorError::InvalidOperation,
                      "custom op name must be at most 128 bytes, got " + std::to_string(n.size()));
  for (unsigned char ch : n) {
    const bool ok = (ch >= 'a' && ch <= 'z') || (ch >= 'A' && ch <= 'Z') || (ch >= '0' && ch <= '9') || ch == '_' ||
                    ch == '.' || ch == ':' || ch == '-';
    if (!ok) throw TensorError(TensorError::InvalidOperation, "custom op name \"" + n + "\" contains unsupported characters");
  }
}
void CustomUnaryRegistry::register_op(const CustomUnaryOp& op) {
  for (const auto& e : ops_)
    if (std::strcmp(e.name(), op.name()) == 0)
      throw TensorError(TensorError::InvalidOperation,
                        std::string("custom unary op \"") + op.name() + "\" is already registered");
  ops_.push_back(op);
}
std::optional<CustomUnaryOp> CustomUnaryRegistry::get(const std::string& name) const {
  for (const auto& e : ops_)
    if (name == e.name()) return e;
  return std::nullopt;
}

// ---- contexts -----------------------------------------------------------------------------------------
// One context (compute stream + collective stream) per device and thread, created on first use
// (heirloom-kernels/src/cuda.rs:7653-7681).
static hl_ctx* context(int ordinal) {
  thread_local std::map<int, hl_ctx*> contexts;
  auto it = contexts.find(ordinal);
  if (it != contexts.end()) return it->second;
  hl_ctx* ctx = nullptr;
  check(hl_ctx_create(ordinal, &ctx));
  contexts[ordinal] = ctx;
  return ctx;
}
RuntimeCounters cuda_runtime_counters(int ordinal) {
  hl_counters_t c;
  std::memset(&c, 0, sizeof(c));
  check(hl_counters_get(context(ordinal), &c));
  RuntimeCounters out;
  out.launches = c.launches;
  out.allocations = c.allocations;
  return out;
}
void synchronize(int ordinal) { check(hl_ctx_sync(context(ordinal))); }

// ---- storage and tensor internals -----------------------------------------------------------------------
struct Storage {
  DType dtype = DType::F32;
  Device device;
  size_t len = 0;
  size_t version = 0;
  std::vector<double> host_f;   // floating dtypes on the host
  std::vector<int64_t> host_i;  // i64 / bool on the host
  hl_buffer* dev = nullptr;     // device storage: f32 (4 bytes) or i64 (8 bytes) per element
  ~Storage() { if (dev) hl_buffer_release(dev); }
  void* ptr() const { return dev ? hl_buffer_ptr(dev) : nullptr; }
};

struct GradFn {
  const char* name = "";
  std::vector<Tensor> inputs;  // where gradients flow
  std::function<std::vector<Tensor>(const Tensor& grad_output)> backward;  // one (possibly undefined) per input
};

struct TensorInner {
  uint64_t id = 0;
  std::shared_ptr<Storage> storage;
  std::vector<size_t> shape, strides;
  size_t offset = 0;
  bool requires_grad = false;
  Tensor grad;
  std::shared_ptr<GradFn> grad_fn;
};

static std::atomic<uint64_t> g_next_id{1};
static thread_local bool g_grad_enabled = true;
bool grad_enabled() { return g_grad_enabled; }
NoGradGuard::NoGradGuard() : previous_(g_grad_enabled) { g_grad_enabled = false; }
NoGradGuard::~NoGradGuard() { g_grad_enabled = previous_; }

static size_t product(const std::vector<size_t>& shape) {
  size_t n = 1;
  for (size_t d : shape) n *= d;
  return n;
}
static std::vector<size_t> contiguous_strides(const std::vector<size_t>& shape) {
  std::vector<size_t> s(shape.size(), 1);
  for (size_t i = shape.size(); i-- > 1;) s[i - 1] = s[i] * shape[i];
  return s;
}
static std::string shape_str(const std::vector<size_t>& shape) {
  std::string s = "[";
  for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
  return s + "]";
}
static Tensor make(std::shared_ptr<Storage> storage, std::vector<size_t> shape, std::vector<size_t> strides, size_t offset) {
  auto inner = std::make_shared<TensorInner>();
  inner->id = g_next_id++;
  inner->storage = std::move(storage);
  inner->shape = std::move(shape);
  inner->strides = std::move(strides);
  inner->offset = offset;
  return Tensor(inner);
}
static Tensor make_contiguous(std::shared_ptr<Storage> storage, const std::vector<size_t>& shape) {
  return make(std::move(storage), shape, contiguous_strides(shape), 0);
}
static std::shared_ptr<Storage> device_storage(DType dtype, int ordinal, size_t len) {
  auto st = std::make_shared<Storage>();
  st->dtype = dtype;
  st->device = Device::cuda(ordinal);
  st->len = len;
  const size_t bytes = std::max<size_t>(len, 1) * (dtype == DType::I64 ? 8 : 4);
  check(hl_buffer_alloc(context(ordinal), bytes, &st->dev));
  return st;
}
static Tensor device_empty(const std::vector<size_t>& shape, int ordinal, DType dtype = DType::F32) {
  return make_contiguous(device_storage(dtype, ordinal, product(shape)), shape);
}
static Tensor device_zeros(const std::vector<size_t>& shape, int ordinal) {
  Tensor t = device_empty(shape, ordinal);
  check(hl_memset_zero(context(ordinal), t.inner()->storage->ptr(), std::max<size_t>(t.numel(), 1) * 4));
  return t;
}

// ---- constructors and accessors -------------------------------------------------------------------------
static void check_len(size_t have, const std::vector<size_t>& shape) {
  if (have != product(shape))
    throw TensorError(TensorError::Shape, "data length " + std::to_string(have) + " does not match shape " + shape_str(shape));
}
Tensor Tensor::from_vec(const std::vector<float>& data, const std::vector<size_t>& shape, bool requires_grad) {
  check_len(data.size(), shape);
  auto st = std::make_shared<Storage>();
  st->dtype = DType::F32;
  st->len = data.size();
  st->host_f.assign(data.begin(), data.end());
  Tensor t = make_contiguous(st, shape);
  t.inner_->requires_grad = requires_grad;
  return t;
}
Tensor Tensor::from_f64(const std::vector<double>& data, const std::vector<size_t>& shape, bool requires_grad) {
  check_len(data.size(), shape);
  auto st = std::make_shared<Storage>();
  st->dtype = DType::F64;
  st->len = data.size();
  st->host_f = data;
  Tensor t = make_contiguous(st, shape);
  t.inner_->requires_grad = requires_grad;
  return t;
}
Tensor Tensor::from_i64(const std::vector<int64_t>& data, const std::vector<size_t>& shape) {
  check_len(data.size(), shape);
  auto st = std::make_shared<Storage>();
  st->dtype = DType::I64;
  st->len = data.size();
  st->host_i = data;
  return make_contiguous(st, shape);
}
Tensor Tensor::zeros(const std::vector<size_t>& shape, DType dtype, Device device) {
  if (device.kind == Device::Cuda) {
    if (dtype != DType::F32) throw TensorError(TensorError::InvalidOperation, "device tensors are created as f32");
    return device_zeros(shape, device.ordinal);
  }
  if (dtype == DType::I64 || dtype == DType::Bool) return from_i64(std::vector<int64_t>(product(shape), 0), shape);
  Tensor t = from_f64(std::vector<double>(product(shape), 0.0), shape);
  t.inner_->storage->dtype = dtype;
  return t;
}
static void need(const Tensor& t) {
  if (!t.defined()) throw TensorError(TensorError::InvalidOperation, "use of an undefined tensor");
}
uint64_t Tensor::id() const { need(*this); return inner_->id; }
const std::vector<size_t>& Tensor::shape() const { need(*this); return inner_->shape; }
const std::vector<size_t>& Tensor::strides() const { need(*this); return inner_->strides; }
size_t Tensor::storage_offset() const { need(*this); return inner_->offset; }
DType Tensor::dtype() const { need(*this); return inner_->storage->dtype; }
Device Tensor::device() const { need(*this); return inner_->storage->device; }
size_t Tensor::numel() const { return product(shape()); }
size_t Tensor::storage_version() const { need(*this); return inner_->storage->version; }
bool Tensor::shares_storage_with(const Tensor& other) const { return inner_->storage == other.inner_->storage; }
bool Tensor::is_contiguous() const {
  size_t expect = 1;
  for (size_t i = shape().size(); i-- > 0;) {
    if (shape()[i] != 1 && strides()[i] != expect) return false;
    expect *= shape()[i];
  }
  return true;
}
bool Tensor::requires_grad() const { need(*this); return inner_->requires_grad; }
bool Tensor::is_leaf() const { need(*this); return !inner_->grad_fn; }
Tensor& Tensor::set_requires_grad(bool on) {
  need(*this);
  if (!is_leaf()) throw TensorError(TensorError::Autograd, "requires_grad can only be changed on leaf tensors");
  if (on && !is_floating(dtype())) throw TensorError(TensorError::Autograd, "only floating tensors can require gradients");
  inner_->requires_grad = on;
  return *this;
}
std::optional<Tensor> Tensor::grad() const {
  need(*this);
  if (!inner_->grad.defined()) return std::nullopt;
  return inner_->grad;
}
std::vector<double> Tensor::grad_f64() const {
  auto g = grad();
  if (!g) throw TensorError(TensorError::Autograd, "tensor has no gradient");
  return g->data_f64();
}
void Tensor::zero_grad() { need(*this); inner_->grad = Tensor(); }
Tensor Tensor::detach() const {
  need(*this);
  return make(inner_->storage, inner_->shape, inner_->strides, inner_->offset);
}

// logical-order walk over a strided tensor
template <typename F>
static void for_each_offset(const Tensor& t, F&& f) {
  const auto& shape = t.shape();
  const auto& strides = t.strides();
  const size_t n = t.numel();
  std::vector<size_t> idx(shape.size(), 0);
  size_t off = t.storage_offset();
  for (size_t i = 0; i < n; ++i) {
    f(off);
    for (size_t d = shape.size(); d-- > 0;) {
      off += strides[d];
      if (++idx[d] < shape[d]) break;
      off -= strides[d] * shape[d];
      idx[d] = 0;
    }
  }
}
std::vector<double> Tensor::data_f64() const {
  need(*this);
  const Storage& st = *inner_->storage;
  std::vector<double> out;
  out.reserve(numel());
  if (st.device.kind == Device::Cuda) {
    if (st.dtype == DType::I64) {
      std::vector<int64_t> raw(std::max<size_t>(st.len, 1));
      check(hl_memcpy_d2h(context(st.device.ordinal), raw.data(), st.ptr(), st.len * 8));
      for_each_offset(*this, [&](size_t o) { out.push_back((double)raw[o]); });
    } else {
      std::vector<float> raw(std::max<size_t>(st.len, 1));
      check(hl_memcpy_d2h(context(st.device.ordinal), raw.data(), st.ptr(), st.len * 4));
      for_each_offset(*this, [&](size_t o) { out.push_back((double)raw[o]); });
    }
  } else if (st.dtype == DType::I64 || st.dtype == DType::Bool) {
    for_each_offset(*this, [&](size_t o) { out.push_back((double)st.host_i[o]); });
  } else {
    for_each_offset(*this, [&](size_t o) { out.push_back(st.host_f[o]); });
  }
  return out;
}
std::vector<float> Tensor::data_f32() const {
  if (dtype() != DType::F32) throw TensorError(TensorError::InvalidOperation, std::string("data_f32 on a ") + dtype_name(dtype()) + " tensor");
  const auto d = data_f64();
  return std::vector<float>(d.begin(), d.end());
}
std::vector<int64_t> Tensor::data_i64() const {
  if (dtype() != DType::I64) throw TensorError(TensorError::InvalidOperation, std::string("data_i64 on a ") + dtype_name(dtype()) + " tensor");
  const auto d = data_f64();
  std::vector<int64_t> out(d.size());
  for (size_t i = 0; i < d.size(); ++i) out[i] = (int64_t)d[i];
  return out;
}
double Tensor::item() const {
  if (numel() != 1) throw TensorError(TensorError::Shape, "item() needs a one-element tensor, got shape " + shape_str(shape()));
  return data_f64()[0];
}

Tensor Tensor::to_device(Device target) const {
  need(*this);
  if (target == device()) return *this;
  Tensor out;
  if (target.kind == Device::Cuda) {
    if (dtype() == DType::I64) {
      const auto host = data_i64();
      out = device_empty(shape(), target.ordinal, DType::I64);
      check(hl_memcpy_h2d(context(target.ordinal), out.inner_->storage->ptr(), host.data(), host.size() * 8));
    } else if (dtype() == DType::F32) {
      const auto host = data_f32();
      out = device_empty(shape(), target.ordinal);
      check(hl_memcpy_h2d(context(target.ordinal), out.inner_->storage->ptr(), host.data(), host.size() * 4));
    } else {
      throw TensorError(TensorError::DeviceError, std::string("device tensors hold f32 or i64, not ") + dtype_name(dtype()));
    }
  } else {
    if (dtype() == DType::I64) out = from_i64(data_i64(), shape());
    else out = from_vec(data_f32(), shape());
  }
  out.inner_->requires_grad = inner_->requires_grad;
  return out;
}

// ---- views ----------------------------------------------------------------------------------------------
static bool record(const std::vector<Tensor>& inputs) {
  if (!g_grad_enabled) return false;
  for (const auto& t : inputs)
    if (t.defined() && t.requires_grad()) return true;
  return false;
}
static Tensor attach(Tensor out, const char* name, std::vector<Tensor> inputs,
                     std::function<std::vector<Tensor>(const Tensor&)> backward) {
  auto fn = std::make_shared<GradFn>();
  fn->name = name;
  fn->inputs = std::move(inputs);
  fn->backward = std::move(backward);
  out.inner()->grad_fn = fn;
  out.inner()->requires_grad = true;
  return out;
}

Tensor Tensor::view(const std::vector<size_t>& new_shape) const {
  need(*this);
  if (!is_contiguous()) throw TensorError(TensorError::Shape, "view requires a contiguous tensor; use reshape");
  if (product(new_shape) != numel())
    throw TensorError(TensorError::Shape, "cannot view shape " + shape_str(shape()) + " as " + shape_str(new_shape));
  Tensor out = make(inner_->storage, new_shape, contiguous_strides(new_shape), inner_->offset);
  if (record({*this})) {
    const std::vector<size_t> old = shape();
    return attach(out, "View", {*this}, [old](const Tensor& g) { return std::vector<Tensor>{g.reshape(old)}; });
  }
  return out;
}
Tensor Tensor::reshape(const std::vector<size_t>& new_shape) const {
  need(*this);
  if (is_contiguous()) return view(new_shape);
  if (product(new_shape) != numel())
    throw TensorError(TensorError::Shape, "cannot reshape " + shape_str(shape()) + " to " + shape_str(new_shape));
  if (device().kind == Device::Cuda)
    throw TensorError(TensorError::DeviceError, "reshape of a non-contiguous device tensor needs a copy, which only host tensors support");
  // host copy in logical order (src/tensor.rs:2464-2496)
  Tensor out = is_floating(dtype()) ? from_f64(data_f64(), new_shape) : from_i64(data_i64(), new_shape);
  out.inner_->storage->dtype = dtype();
  return out;
}
Tensor Tensor::permute(const std::vector<size_t>& dims) const {
  need(*this);
  if (dims.size() != ndim()) throw TensorError(TensorError::Shape, "permute needs one entry per dimension");
  std::vector<bool> seen(ndim(), false);
  std::vector<size_t> sh(ndim()), st(ndim());
  for (size_t i = 0; i < dims.size(); ++i) {
    if (dims[i] >= ndim() || seen[dims[i]]) throw TensorError(TensorError::Shape, "permute dimensions must be a permutation");
    seen[dims[i]] = true;
    sh[i] = shape()[dims[i]];
    st[i] = strides()[dims[i]];
  }
  Tensor out = make(inner_->storage, sh, st, inner_->offset);
  if (record({*this})) {
    std::vector<size_t> inverse(dims.size());
    for (size_t i = 0; i < dims.size(); ++i) inverse[dims[i]] = i;
    return attach(out, "Permute", {*this}, [inverse](const Tensor& g) { return std::vector<Tensor>{g.permute(inverse)}; });
  }
  return out;
}
Tensor Tensor::transpose(size_t dim0, size_t dim1) const {
  need(*this);
  if (dim0 >= ndim() || dim1 >= ndim())
    throw TensorError(TensorError::Shape, "transpose dimensions out of range for rank " + std::to_string(ndim()));
  std::vector<size_t> dims(ndim());
  std::iota(dims.begin(), dims.end(), 0);
  std::swap(dims[dim0], dims[dim1]);
  return permute(dims);
}
Tensor Tensor::narrow(size_t dim, size_t start, size_t length) const {
  need(*this);
  if (dim >= ndim() || start + length > shape()[dim])
    throw TensorError(TensorError::Shape, "narrow range " + std::to_string(start) + ".." + std::to_string(start + length) +
                                              " exceeds dimension of size " + (dim < ndim() ? std::to_string(shape()[dim]) : "?"));
  std::vector<size_t> sh = shape();
  sh[dim] = length;
  Tensor out = make(inner_->storage, sh, strides(), inner_->offset + start * strides()[dim]);
  if (record({*this})) {
    const Tensor self = *this;
    return attach(out, "Narrow", {*this}, [self, dim, start, length](const Tensor& g) {
      // the gradient of the full tensor is zero outside the slice
      if (self.device().kind != Device::Cuda || !self.is_contiguous() || dim != 0 || !g.is_contiguous())
        throw TensorError(TensorError::Autograd, "narrow backward is supported for slices of the first dimension of contiguous device tensors");
      Tensor full = device_zeros(self.shape(), self.device().ordinal);
      const size_t row = self.numel() / std::max<size_t>(self.shape()[0], 1);
      float* dst = static_cast<float*>(full.inner()->storage->ptr()) + start * row;
      const float* src = static_cast<const float*>(g.inner()->storage->ptr()) + g.storage_offset();
      check(hl_scale_f32(context(self.device().ordinal), src, 1.0f, dst, length * row));
      return std::vector<Tensor>{full};
    });
  }
  return out;
}
Tensor Tensor::expand(const std::vector<size_t>& new_shape) const {
  need(*this);
  if (new_shape.size() < ndim()) throw TensorError(TensorError::Shape, "expand cannot drop dimensions");
  const size_t lead = new_shape.size() - ndim();
  std::vector<size_t> st(new_shape.size(), 0);
  for (size_t i = 0; i < ndim(); ++i) {
    if (shape()[i] == new_shape[lead + i]) st[lead + i] = strides()[i];
    else if (shape()[i] == 1) st[lead + i] = 0;
    else throw TensorError(TensorError::Shape, "cannot expand " + shape_str(shape()) + " to " + shape_str(new_shape));
  }
  Tensor out = make(inner_->storage, new_shape, st, inner_->offset);
  if (record({*this})) {
    const Tensor self = *this;
    return attach(out, "Expand", {*this}, [self](const Tensor& g) {
      // supported form: a [cols] vector expanded over rows; its gradient is the column sum
      if (self.ndim() != 1 || g.ndim() != 2 || !g.is_contiguous() || g.device().kind != Device::Cuda)
        throw TensorError(TensorError::Autograd, "expand backward is supported for a vector expanded over rows on the device");
      Tensor out = device_empty(self.shape(), g.device().ordinal);
      check(hl_bias_grad(context(g.device().ordinal), static_cast<const float*>(g.inner()->storage->ptr()) + g.storage_offset(),
                         HL_F32, static_cast<float*>(out.inner()->storage->ptr()), (int)g.shape()[0], (int)g.shape()[1]));
      return std::vector<Tensor>{out};
    });
  }
  return out;
}

// ---- device op helpers ----------------------------------------------------------------------------------
static int cuda_ordinal(const Tensor& t, const char* op) {
  if (t.device().kind != Device::Cuda)
    throw TensorError(TensorError::DeviceError, std::string(op) + " runs on the GPU only: move the tensor with to_device(Device::cuda(n)) first");
  return t.device().ordinal;
}
static void same_device(const Tensor& a, const Tensor& b, const char* op) {
  if (a.device() != b.device()) throw TensorError(TensorError::DeviceError, std::string(op) + ": operands are on different devices");
}
static void need_f32(const Tensor& t, const char* op) {
  if (t.dtype() != DType::F32) throw TensorError(TensorError::InvalidOperation, std::string(op) + " expects f32 device tensors, got " + dtype_name(t.dtype()));
}
// CUDA ops demand contiguous storage (src/tensor.rs:1122-1151)
static const float* fptr(const Tensor& t, const char* op) {
  need_f32(t, op);
  if (!t.is_contiguous()) throw TensorError(TensorError::DeviceError, std::string(op) + ": device kernels need a contiguous tensor");
  return static_cast<const float*>(t.inner()->storage->ptr()) + t.storage_offset();
}
static float* fptr_mut(Tensor& t) { return static_cast<float*>(t.inner()->storage->ptr()) + t.storage_offset(); }
static hl_matrix_layout layout_of(const Tensor& t) {  // MatrixLayout (cuda.rs:536-560)
  hl_matrix_layout l;
  l.rows = (long long)t.shape()[0];
  l.cols = (long long)t.shape()[1];
  l.row_stride = (long long)t.strides()[0];
  l.col_stride = (long long)t.strides()[1];
  l.offset = (long long)t.storage_offset();
  return l;
}
static hl_matrix_layout transposed(hl_matrix_layout l) {
  std::swap(l.rows, l.cols);
  std::swap(l.row_stride, l.col_stride);
  return l;
}
// A fresh buffer with the memory arrangement of `like` when that is a dense permutation of a
// contiguous tensor, so that undoing the view yields a contiguous gradient; contiguous otherwise.
static Tensor empty_with_layout_of(const Tensor& like) {
  const int ordinal = like.device().ordinal;
  std::vector<size_t> order(like.ndim());
  std::iota(order.begin(), order.end(), 0);
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return like.strides()[a] > like.strides()[b]; });
  size_t expect = 1;
  bool dense = true;
  for (size_t i = order.size(); i-- > 0;) {
    if (like.shape()[order[i]] != 1 && like.strides()[order[i]] != expect) dense = false;
    expect *= like.shape()[order[i]];
  }
  if (!dense) return device_empty(like.shape(), ordinal);
  return make(device_storage(DType::F32, ordinal, like.numel()), like.shape(), like.strides(), 0);
}

// ---- ops ------------------------------------------------------------------------------------------------
static Tensor binary(const Tensor& a, const Tensor& b, int op, const char* name) {
  const int ordinal = cuda_ordinal(a, name);
  same_device(a, b, name);
  hl_ctx* ctx = context(ordinal);
  const bool bias_form = op == HL_ADD && a.ndim() == 2 && b.ndim() == 1 && b.shape()[0] == a.shape()[1];
  if (!bias_form && a.shape() != b.shape())
    throw TensorError(TensorError::Shape, std::string(name) + ": shapes " + shape_str(a.shape()) + " and " + shape_str(b.shape()) +
                                              " are neither equal nor [rows, cols] + [cols]");
  Tensor out = device_empty(a.shape(), ordinal);
  if (bias_form) check(hl_bias_add_f32(ctx, fptr(a, name), fptr(b, name), fptr_mut(out), (int)a.shape()[0], (int)a.shape()[1]));
  else check(hl_binary_f32(ctx, op, fptr(a, name), fptr(b, name), fptr_mut(out), a.numel()));
  if (!record({a, b})) return out;
  return attach(out, name, {a, b}, [a, b, op, bias_form, ordinal](const Tensor& g) {
    hl_ctx* ctx = context(ordinal);
    std::vector<Tensor> grads(2);
    const float* gp = fptr(g, "binary backward");
    if (a.requires_grad()) {
      if (op == HL_ADD || op == HL_SUB) grads[0] = g;
      else {
        grads[0] = device_empty(a.shape(), ordinal);
        check(hl_binary_f32(ctx, op == HL_MUL ? HL_MUL : HL_DIV, gp, fptr(b, "binary backward"), fptr_mut(grads[0]), a.numel()));
      }
    }
    if (b.requires_grad()) {
      if (bias_form) {
        grads[1] = device_empty(b.shape(), ordinal);
        check(hl_bias_grad(ctx, gp, HL_F32, fptr_mut(grads[1]), (int)a.shape()[0], (int)a.shape()[1]));
      } else if (op == HL_ADD) {
        grads[1] = g;
      } else if (op == HL_SUB) {
        grads[1] = device_empty(b.shape(), ordinal);
        check(hl_scale_f32(ctx, gp, -1.0f, fptr_mut(grads[1]), b.numel()));
      } else if (op == HL_MUL) {
        grads[1] = device_empty(b.shape(), ordinal);
        check(hl_binary_f32(ctx, HL_MUL, gp, fptr(a, "binary backward"), fptr_mut(grads[1]), b.numel()));
      } else {  // d(a/b)/db = -a/b^2 * g
        Tensor q = device_empty(b.shape(), ordinal), r = device_empty(b.shape(), ordinal);
        check(hl_binary_f32(ctx, HL_DIV, fptr(a, "div"), fptr(b, "div"), fptr_mut(q), b.numel()));
        check(hl_binary_f32(ctx, HL_DIV, fptr(q, "div"), fptr(b, "div"), fptr_mut(r), b.numel()));
        check(hl_binary_f32(ctx, HL_MUL, fptr(r, "div"), gp, fptr_mut(q), b.numel()));
        grads[1] = device_empty(b.shape(), ordinal);
        check(hl_scale_f32(ctx, fptr(q, "div"), -1.0f, fptr_mut(grads[1]), b.numel()));
      }
    }
    return grads;
  });
}
Tensor Tensor::add(const Tensor& o) const { return binary(*this, o, HL_ADD, "add"); }
Tensor Tensor::sub(const Tensor& o) const { return binary(*this, o, HL_SUB, "sub"); }
Tensor Tensor::mul(const Tensor& o) const { return binary(*this, o, HL_MUL, "mul"); }
Tensor Tensor::div(const Tensor& o) const { return binary(*this, o, HL_DIV, "div"); }

Tensor Tensor::matmul(const Tensor& other) const {
  const int ordinal = cuda_ordinal(*this, "matmul");
  same_device(*this, other, "matmul");
  need_f32(*this, "matmul");
  need_f32(other, "matmul");
  if (ndim() != 2 || other.ndim() != 2)
    throw TensorError(TensorError::Shape, "matmul on the device takes rank-2 operands, got " + shape_str(shape()) + " and " + shape_str(other.shape()));
  if (shape()[1] != other.shape()[0])
    throw TensorError(TensorError::Shape, "matmul inner dimensions differ: " + shape_str(shape()) + " x " + shape_str(other.shape()));
  const Tensor a = *this, b = other;
  Tensor out = device_empty({shape()[0], other.shape()[1]}, ordinal);
  const hl_matrix_layout la = layout_of(a), lb = layout_of(b), lo = layout_of(out);
  check(hl_matmul_f32_strided(context(ordinal), static_cast<const float*>(a.inner()->storage->ptr()), &la,
                              static_cast<const float*>(b.inner()->storage->ptr()), &lb,
                              static_cast<float*>(out.inner()->storage->ptr()), &lo, 0));
  if (!record({a, b})) return out;
  return attach(out, "Matmul", {a, b}, [a, b, ordinal](const Tensor& g) {
    // dA = dY·Bᵀ, dB = Aᵀ·dY (src/tensor/autograd.rs:2012-2104); each gradient takes the memory
    // arrangement of its operand
    hl_ctx* ctx = context(ordinal);
    std::vector<Tensor> grads(2);
    const hl_matrix_layout lg = layout_of(g);
    const float* gp = static_cast<const float*>(g.inner()->storage->ptr());
    if (a.requires_grad()) {
      grads[0] = empty_with_layout_of(a);
      const hl_matrix_layout lbt = transposed(layout_of(b)), lo = layout_of(grads[0]);
      check(hl_matmul_f32_strided(ctx, gp, &lg, static_cast<const float*>(b.inner()->storage->ptr()), &lbt,
                                  static_cast<float*>(grads[0].inner()->storage->ptr()), &lo, 0));
    }
    if (b.requires_grad()) {
      grads[1] = empty_with_layout_of(b);
      const hl_matrix_layout lat = transposed(layout_of(a)), lo = layout_of(grads[1]);
      check(hl_matmul_f32_strided(ctx, static_cast<const float*>(a.inner()->storage->ptr()), &lat, gp, &lg,
                                  static_cast<float*>(grads[1].inner()->storage->ptr()), &lo, 0));
    }
    return grads;
  });
}

Tensor Tensor::relu() const {
  const int ordinal = cuda_ordinal(*this, "relu");
  const Tensor x = *this;
  Tensor out = device_empty(shape(), ordinal);
  check(hl_relu_f32(context(ordinal), fptr(x, "relu"), fptr_mut(out), numel()));
  if (!record({x})) return out;
  return attach(out, "Relu", {x}, [x, ordinal](const Tensor& g) {
    Tensor gx = device_empty(x.shape(), ordinal);
    check(hl_relu_backward_f32(context(ordinal), fptr(x, "relu"), fptr(g, "relu backward"), fptr_mut(gx), x.numel()));
    return std::vector<Tensor>{gx};
  });
}
Tensor Tensor::gelu() const {
  const int ordinal = cuda_ordinal(*this, "gelu");
  const Tensor x = *this;
  Tensor out = device_empty(shape(), ordinal);
  check(hl_gelu(context(ordinal), fptr(x, "gelu"), fptr_mut(out), HL_F32, numel()));
  if (!record({x})) return out;
  return attach(out, "Gelu", {x}, [x, ordinal](const Tensor& g) {
    Tensor gx = device_empty(x.shape(), ordinal);
    check(hl_gelu_backward(context(ordinal), fptr(x, "gelu"), fptr(g, "gelu backward"), fptr_mut(gx), HL_F32, x.numel()));
    return std::vector<Tensor>{gx};
  });
}
Tensor Tensor::softmax_dim(size_t dim) const {
  const int ordinal = cuda_ordinal(*this, "softmax_dim");
  if (ndim() != 2 || dim != 1) throw TensorError(TensorError::Shape, "softmax_dim on the device takes a rank-2 tensor and its last dimension");
  const Tensor x = *this;
  Tensor out = device_empty(shape(), ordinal);
  check(hl_softmax_rows_f32(context(ordinal), fptr(x, "softmax_dim"), fptr_mut(out), (int)shape()[0], (int)shape()[1]));
  if (!record({x})) return out;
  const Tensor y = out.detach();
  return attach(out, "SoftmaxDim", {x}, [y, ordinal](const Tensor& g) {
    Tensor gx = device_empty(y.shape(), ordinal);
    check(hl_softmax_rows_backward_f32(context(ordinal), fptr(y, "softmax"), fptr(g, "softmax backward"), fptr_mut(gx),
                                       (int)y.shape()[0], (int)y.shape()[1]));
    return std::vector<Tensor>{gx};
  });
}
static Tensor reduce_all(const Tensor& x, bool mean) {
  const char* name = mean ? "mean" : "sum";
  const int ordinal = cuda_ordinal(x, name);
  Tensor out = device_empty({}, ordinal);
  if (mean) check(hl_mean_f32(context(ordinal), fptr(x, name), x.numel(), fptr_mut(out)));
  else check(hl_sum_f32(context(ordinal), fptr(x, name), x.numel(), fptr_mut(out)));
  if (!record({x})) return out;
  return attach(out, mean ? "Mean" : "Sum", {x}, [x, mean, ordinal](const Tensor& g) {
    const double scale = mean ? 1.0 / (double)std::max<size_t>(x.numel(), 1) : 1.0;
    Tensor gx = device_empty(x.shape(), ordinal);
    check(hl_fill_f32(context(ordinal), fptr_mut(gx), (float)(g.item() * scale), x.numel()));
    return std::vector<Tensor>{gx};
  });
}
Tensor Tensor::sum() const { return reduce_all(*this, false); }
Tensor Tensor::mean() const { return reduce_all(*this, true); }

Tensor Tensor::layer_norm_last_dim(const Tensor& weight, const Tensor& bias, double eps) const {
  const int ordinal = cuda_ordinal(*this, "layer_norm_last_dim");
  same_device(*this, weight, "layer_norm_last_dim");
  same_device(*this, bias, "layer_norm_last_dim");
  if (ndim() < 1) throw TensorError(TensorError::Shape, "layer_norm_last_dim needs at least one dimension");
  const size_t feat = shape().back();
  if (weight.numel() != feat || bias.numel() != feat)
    throw TensorError(TensorError::Shape, "layer_norm_last_dim: weight and bias must have " + std::to_string(feat) + " elements");
  const size_t rows = numel() / std::max<size_t>(feat, 1);
  const Tensor x = *this;
  Tensor out = device_empty(shape(), ordinal), mean = device_empty({rows}, ordinal), rstd = device_empty({rows}, ordinal);
  check(hl_layer_norm_forward(context(ordinal), fptr(x, "layer_norm"), HL_F32, fptr(weight, "layer_norm"), fptr(bias, "layer_norm"),
                              fptr_mut(out), HL_F32, fptr_mut(mean), fptr_mut(rstd), (int)rows, (int)feat, (float)eps));
  if (!record({x, weight, bias})) return out;
  return attach(out, "LayerNormLastDim", {x, weight, bias}, [x, weight, mean, rstd, rows, feat, ordinal](const Tensor& g) {
    Tensor dx = device_empty(x.shape(), ordinal), dw = device_empty({feat}, ordinal), db = device_empty({feat}, ordinal);
    check(hl_layer_norm_backward(context(ordinal), fptr(x, "layer_norm"), HL_F32, fptr(weight, "layer_norm"), fptr(g, "layer_norm backward"),
                                 fptr(mean, "layer_norm"), fptr(rstd, "layer_norm"), nullptr, fptr_mut(dx), nullptr, fptr_mut(dw),
                                 fptr_mut(db), nullptr, (int)rows, (int)feat));
    return std::vector<Tensor>{dx, dw, db};
  });
}

Tensor Tensor::embedding(const Tensor& weight, const Tensor& indices) {
  const int ordinal = cuda_ordinal(weight, "embedding");
  same_device(weight, indices, "embedding");
  if (indices.dtype() != DType::I64) throw TensorError(TensorError::InvalidOperation, "embedding indices must be i64");
  if (weight.ndim() != 2) throw TensorError(TensorError::Shape, "embedding weight must be rank 2");
  if (!indices.is_contiguous()) throw TensorError(TensorError::DeviceError, "embedding: device kernels need contiguous indices");
  const size_t n = indices.numel(), dim = weight.shape()[1], rows = weight.shape()[0];
  std::vector<size_t> out_shape = indices.shape();
  out_shape.push_back(dim);
  Tensor out = device_empty(out_shape, ordinal);
  const int64_t* idx = static_cast<const int64_t*>(indices.inner()->storage->ptr()) + indices.storage_offset();
  check(hl_embedding_forward(context(ordinal), fptr(weight, "embedding"), (int)rows, idx, nullptr, 0, fptr_mut(out), HL_F32, (int)n, (int)dim));
  if (!record({weight})) return out;
  return attach(out, "Embedding", {weight}, [weight, indices, idx, n, dim, rows, ordinal](const Tensor& g) {
    Tensor gw = device_zeros(weight.shape(), ordinal);  // repeats accumulate (src/tensor/autograd.rs:2234-2261)
    check(hl_embedding_backward(context(ordinal), fptr(g, "embedding backward"), idx, fptr_mut(gw), (int)rows, nullptr, 0, (int)n, (int)dim));
    return std::vector<Tensor>{gw};
  });
}

Tensor Tensor::causal_self_attention(const Tensor& q, const Tensor& k, const Tensor& v, size_t n_heads) {
  const int ordinal = cuda_ordinal(q, "causal_self_attention");
  same_device(q, k, "causal_self_attention");
  same_device(q, v, "causal_self_attention");
  if (n_heads == 0) throw TensorError(TensorError::InvalidOperation, "causal_self_attention requires n_heads > 0");
  if (q.ndim() != 3 || q.shape() != k.shape() || q.shape() != v.shape())
    throw TensorError(TensorError::Shape, "causal_self_attention takes q, k, v of one shape [batch, time, channels]");
  const size_t B = q.shape()[0], T = q.shape()[1], C = q.shape()[2];
  if (C % n_heads != 0) throw TensorError(TensorError::Shape, "channels " + std::to_string(C) + " are not divisible by n_heads " + std::to_string(n_heads));
  Tensor out = device_empty(q.shape(), ordinal), probs = device_empty({B, n_heads, T, T}, ordinal);
  check(hl_causal_attention_f32_forward(context(ordinal), fptr(q, "attention"), fptr(k, "attention"), fptr(v, "attention"), fptr_mut(out),
                                        fptr_mut(probs), (int)B, (int)T, (int)C, (int)n_heads));
  if (!record({q, k, v})) return out;
  return attach(out, "CausalSelfAttention", {q, k, v}, [q, k, v, probs, B, T, C, n_heads, ordinal](const Tensor& g) {
    Tensor dq = device_empty(q.shape(), ordinal), dk = device_empty(q.shape(), ordinal), dv = device_empty(q.shape(), ordinal);
    check(hl_causal_attention_f32_backward(context(ordinal), fptr(q, "attention"), fptr(k, "attention"), fptr(v, "attention"),
                                           fptr(probs, "attention"), fptr(g, "attention backward"), fptr_mut(dq), fptr_mut(dk), fptr_mut(dv),
                                           (int)B, (int)T, (int)C, (int)n_heads));
    return std::vector<Tensor>{dq, dk, dv};
  });
}

Tensor Tensor::cross_entropy_for_logits(const Tensor& targets) const {
  const int ordinal = cuda_ordinal(*this, "cross_entropy_for_logits");
  same_device(*this, targets, "cross_entropy_for_logits");
  if (ndim() != 2) throw TensorError(TensorError::Shape, "cross_entropy_for_logits takes [rows, classes] logits");
  if (targets.dtype() != DType::I64 || targets.numel() != shape()[0] || !targets.is_contiguous())
    throw TensorError(TensorError::Shape, "cross_entropy_for_logits takes one contiguous i64 target per row");
  const Tensor z = *this;
  const size_t rows = shape()[0], classes = shape()[1];
  const bool rec = record({z});
  Tensor loss = device_empty({}, ordinal);
  Tensor dlogits = rec ? device_empty(shape(), ordinal) : Tensor();
  const int64_t* tg = static_cast<const int64_t*>(targets.inner()->storage->ptr()) + targets.storage_offset();
  check(hl_cross_entropy(context(ordinal), fptr(z, "cross_entropy"), (long long)classes, tg, (int)rows, (int)classes, 1.0f, fptr_mut(loss),
                         nullptr, rec ? fptr_mut(dlogits) : nullptr, HL_F32, (long long)classes));
  if (!rec) return loss;
  return attach(loss, "CrossEntropyForLogits", {z}, [dlogits, targets, ordinal](const Tensor& g) {
    const double scale = g.item();
    if (scale == 1.0) return std::vector<Tensor>{dlogits};
    Tensor out = device_empty(dlogits.shape(), ordinal);
    check(hl_scale_f32(context(ordinal), fptr(dlogits, "cross_entropy"), (float)scale, fptr_mut(out), dlogits.numel()));
    return std::vector<Tensor>{out};
  });
}

// Host callbacks over f64 slices; a device tensor is staged through the host
// (src/tensor.rs:4496-4519).
Tensor Tensor::apply_custom_unary(const CustomUnaryOp& op) const {
  need(*this);
  if (!is_floating(dtype()))
    throw TensorError(TensorError::InvalidOperation, std::string("custom unary op ") + op.name() + " requires a floating tensor, got " + dtype_name(dtype()));
  const Tensor x = *this;
  const std::vector<double> input = data_f64();
  const std::vector<size_t> shp = shape();
  const CustomUnaryForwardContext fctx{op.name(), input, shp, dtype(), device()};
  std::vector<double> output = op.forward_fn()(fctx);
  if (output.size() != input.size())
    throw TensorError(TensorError::InvalidOperation, std::string("custom unary op ") + op.name() + " returned " + std::to_string(output.size()) +
                                                         " elements for an input of " + std::to_string(input.size()));
  Tensor out;
  if (dtype() == DType::F64) out = from_f64(output, shp);
  else {
    out = from_vec(std::vector<float>(output.begin(), output.end()), shp);
    if (device().kind == Device::Cuda) out = out.to_device(device());
  }
  if (!record({x})) return out;
  const DType dt = dtype();
  const Device dev = device();
  return attach(out, "CustomUnary", {x}, [x, op, input, output, shp, dt, dev](const Tensor& g) {
    const std::vector<double> go = g.data_f64();
    const CustomUnaryBackwardContext bctx{op.name(), input, output, go, shp, dt, dev};
    const std::vector<double> gi = op.backward_fn()(bctx);
    if (gi.size() != input.size())
      throw TensorError(TensorError::Autograd, std::string("custom unary op ") + op.name() + " returned gradient length " +
                                                   std::to_string(gi.size()) + " for an input of " + std::to_string(input.size()));
    Tensor gx = dt == DType::F64 ? Tensor::from_f64(gi, shp) : Tensor::from_vec(std::vector<float>(gi.begin(), gi.end()), shp);
    if (dev.kind == Device::Cuda) gx = gx.to_device(dev);
    return std::vector<Tensor>{gx};
  });
}

// ---- autograd driver --------------------------------------------------------------------------------------
// First gradient adopts the buffer, later ones are added (src/tensor.rs:1721-1846).
static void accumulate(std::unordered_map<TensorInner*, Tensor>& pending, const Tensor& target, const Tensor& grad) {
  if (grad.shape() != target.shape())
    throw TensorError(TensorError::Autograd, "gradient shape " + shape_str(grad.shape()) + " does not match tensor shape " + shape_str(target.shape()));
  auto it = pending.find(target.inner().get());
  if (it == pending.end()) {
    pending[target.inner().get()] = grad;
    return;
  }
  Tensor& have = it->second;
  if (have.device().kind != Device::Cuda || !have.is_contiguous() || !grad.is_contiguous())
    throw TensorError(TensorError::Autograd, "adding gradients needs contiguous device tensors");
  const int ordinal = have.device().ordinal;
  Tensor sum = device_empty(have.shape(), ordinal);
  check(hl_binary_f32(context(ordinal), HL_ADD, fptr(have, "grad accumulate"), fptr(grad, "grad accumulate"), fptr_mut(sum), have.numel()));
  have = sum;
}

void Tensor::backward() const {
  need(*this);
  if (numel() != 1) throw TensorError(TensorError::Autograd, "backward() needs a one-element tensor, got shape " + shape_str(shape()));
  if (!requires_grad()) throw TensorError(TensorError::Autograd, "backward() on a tensor that does not require gradients");
  // depth-first topological order (src/tensor/autograd.rs:2922-2943)
  std::vector<Tensor> order;
  std::unordered_set<TensorInner*> visited;
  std::vector<std::pair<Tensor, size_t>> stack{{*this, 0}};
  visited.insert(inner_.get());
  while (!stack.empty()) {
    auto& [node, next] = stack.back();
    const auto& fn = node.inner()->grad_fn;
    if (fn && next < fn->inputs.size()) {
      const Tensor child = fn->inputs[next++];
      if (child.defined() && child.requires_grad() && visited.insert(child.inner().get()).second) stack.push_back({child, 0});
    } else {
      order.push_back(node);
      stack.pop_back();
    }
  }
  std::unordered_map<TensorInner*, Tensor> pending;
  Tensor seed;
  if (device().kind == Device::Cuda) {
    seed = device_empty(shape(), device().ordinal);
    check(hl_fill_f32(context(device().ordinal), fptr_mut(seed), 1.0f, 1));
  } else {
    seed = dtype() == DType::F64 ? from_f64({1.0}, shape()) : from_vec({1.0f}, shape());
  }
  pending[inner_.get()] = seed;
  NoGradGuard guard;  // the backward pass records no graph of its own
  for (size_t i = order.size(); i-- > 0;) {
    Tensor node = order[i];
    auto it = pending.find(node.inner().get());
    if (it == pending.end()) continue;
    const Tensor grad = it->second;
    pending.erase(it);
    const auto fn = node.inner()->grad_fn;
    if (!fn) {  // leaf: keep the gradient, adding to one left by an earlier backward
      if (node.inner()->grad.defined()) {
        std::unordered_map<TensorInner*, Tensor> tmp{{node.inner().get(), node.inner()->grad}};
        accumulate(tmp, node, grad);
        node.inner()->grad = tmp[node.inner().get()];
      } else {
        node.inner()->grad = grad;
      }
      continue;
    }
    const std::vector<Tensor> grads = fn->backward(grad);
    if (grads.size() != fn->inputs.size()) throw TensorError(TensorError::Autograd, std::string(fn->name) + " returned the wrong number of gradients");
    for (size_t j = 0; j < grads.size(); ++j)
      if (grads[j].defined() && fn->inputs[j].defined() && fn->inputs[j].requires_grad()) accumulate(pending, fn->inputs[j], grads[j]);
    node.inner()->grad_fn.reset();  // the graph is released as the walk passes (non-leaf gradients are not kept)
  }
}

// ---- modules ------------------------------------------------------------------------------------------------
namespace nn {

Tensor Linear::forward(const Tensor& x) const {
  Tensor y = x.matmul(weight.transpose(0, 1));
  return bias.defined() ? y.add(bias) : y;
}
Tensor CausalSelfAttention::forward(const Tensor& x, size_t batch, size_t time) const {
  const size_t d = x.shape()[1];
  const Tensor q = q_proj.forward(x).reshape({batch, time, d});
  const Tensor k = k_proj.forward(x).reshape({batch, time, d});
  const Tensor v = v_proj.forward(x).reshape({batch, time, d});
  const Tensor o = Tensor::causal_self_attention(q, k, v, n_heads).reshape({batch * time, d});
  return out_proj.forward(o);
}
static void append(std::vector<Tensor>& to, const std::vector<Tensor>& from) { to.insert(to.end(), from.begin(), from.end()); }
std::vector<Tensor> CausalSelfAttention::parameters() const {
  std::vector<Tensor> p;
  append(p, q_proj.parameters()); append(p, k_proj.parameters()); append(p, v_proj.parameters()); append(p, out_proj.parameters());
  return p;
}
std::vector<Tensor> FeedForward::parameters() const {
  std::vector<Tensor> p = fc1.parameters();
  append(p, fc2.parameters());
  return p;
}
Tensor TransformerBlock::forward(const Tensor& x, size_t batch, size_t time) const {
  const Tensor r = x.add(attention.forward(ln1.forward(x), batch, time));
  return r.add(feed_forward.forward(ln2.forward(r)));
}
std::vector<Tensor> TransformerBlock::parameters() const {
  std::vector<Tensor> p = ln1.parameters();
  append(p, attention.parameters()); append(p, ln2.parameters()); append(p, feed_forward.parameters());
  return p;
}

AdamW::AdamW(std::vector<Tensor> parameters, double lr, double beta1, double beta2, double eps, double weight_decay,
             std::optional<double> clip_norm)
    : params_(std::move(parameters)), lr_(lr), beta1_(beta1), beta2_(beta2), eps_(eps), weight_decay_(weight_decay), clip_norm_(clip_norm) {
  for (const auto& p : params_) {
    if (p.device().kind != Device::Cuda || p.dtype() != DType::F32 || !p.is_contiguous())
      throw TensorError(TensorError::InvalidOperation, "AdamW takes contiguous f32 device parameters");
    m_.push_back(device_zeros(p.shape(), p.device().ordinal));
    v_.push_back(device_zeros(p.shape(), p.device().ordinal));
  }
}
void AdamW::zero_grad() { for (auto& p : params_) p.zero_grad(); }
void AdamW::step() {
  // clip = max_norm/(‖g‖+1e-12) when the global norm exceeds max_norm (src/nn.rs:2589-2665)
  double clip = 1.0;
  if (clip_norm_) {
    double sum_sq = 0.0;
    for (const auto& p : params_) {
      auto g = p.grad();
      if (!g) continue;
      Tensor s = device_empty({}, p.device().ordinal);
      check(hl_sum_squares_f32(context(p.device().ordinal), fptr(*g, "clip"), g->numel(), fptr_mut(s)));
      sum_sq += s.item();
    }
    const double norm = std::sqrt(sum_sq);
    if (norm > *clip_norm_) clip = *clip_norm_ / (norm + 1e-12);
  }
  step_ += 1;  // once per call, also when no parameter has a gradient
  hl_adamw_params hp;
  hp.lr = (float)lr_; hp.beta1 = (float)beta1_; hp.beta2 = (float)beta2_; hp.eps = (float)eps_;
  hp.weight_decay = (float)weight_decay_; hp.clip_scale = (float)clip;
  hp.bias_correction1 = (float)(1.0 - std::pow(beta1_, step_));  // host f64 -> f32 (src/nn.rs:2467-2505)
  hp.bias_correction2 = (float)(1.0 - std::pow(beta2_, step_));
  for (size_t i = 0; i < params_.size(); ++i) {
    auto g = params_[i].grad();
    if (!g) continue;  // parameters without a gradient are skipped
    Tensor& p = params_[i];
    check(hl_adamw_f32(context(p.device().ordinal), fptr_mut(p), fptr(*g, "AdamW"), fptr_mut(m_[i]), fptr_mut(v_[i]), p.numel(), &hp));
    p.inner()->storage->version += 1;
  }
}

}  // namespace nn
}  // namespace heirloom
