// Test driver of the host-side tensor interface.  Modes:
//   host_tests cpu                 checks that need no GPU (catalog, custom-op rules, views, error routing)
//   host_tests gpu                 device checks with closed-form expectations
//   host_tests decoder IN OUT      one training step of a small decoder built from the nn modules; IN holds the
//                                  configuration, parameters and tokens, OUT receives loss, gradients and the
//                                  parameters after one AdamW step (the Python test compares them with the oracle)
// The scenarios follow the reference's own tests: tests/operator_registry.rs, tests/custom_ops.rs,
// tests/tensor_ops.rs (views), tests/transformer_runtime.rs:1460-1473 (embedding gradients).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>

#include "heirloom.hpp"

using namespace heirloom;

static int g_failures = 0;
#define EXPECT(cond)                                                                 \
  do {                                                                               \
    if (!(cond)) {                                                                   \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);                    \
      ++g_failures;                                                                  \
    }                                                                                \
  } while (0)
template <typename F>
static bool throws_with(F&& f, const char* needle) {
  try {
    f();
  } catch (const TensorError& e) {
    if (std::strstr(e.what(), needle)) return true;
    std::printf("  wrong message: %s\n", e.what());
    return false;
  }
  return false;
}
static bool close(const std::vector<double>& a, const std::vector<double>& b, double tol) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (std::fabs(a[i] - b[i]) > tol * std::max(1.0, std::fabs(b[i]))) {
      std::printf("  index %zu: %.9g vs %.9g\n", i, a[i], b[i]);
      return false;
    }
  return true;
}

static std::vector<double> square_forward(const CustomUnaryForwardContext& c) {
  std::vector<double> out;
  for (double v : c.input) out.push_back(v * v);
  return out;
}
static std::vector<double> square_backward(const CustomUnaryBackwardContext& c) {
  std::vector<double> out;
  for (size_t i = 0; i < c.input.size(); ++i) out.push_back(2.0 * c.input[i] * c.grad_output[i]);
  return out;
}
static std::vector<double> cubic_forward(const CustomUnaryForwardContext& c) {
  std::vector<double> out;
  for (double v : c.input) out.push_back((v + 1.0) * (v + 1.0) * (v + 1.0));
  return out;
}
static std::vector<double> cubic_backward(const CustomUnaryBackwardContext& c) {
  std::vector<double> out;
  for (size_t i = 0; i < c.input.size(); ++i) out.push_back(3.0 * (c.input[i] + 1.0) * (c.input[i] + 1.0) * c.grad_output[i]);
  return out;
}
static std::vector<double> bad_forward(const CustomUnaryForwardContext& c) { return std::vector<double>(c.input.size() + 1, 0.0); }
static std::vector<double> bad_backward(const CustomUnaryBackwardContext&) { return {1.0}; }

// ---- no GPU --------------------------------------------------------------------------------------------
static void cpu_tests() {
  // tests/operator_registry.rs
  const auto& catalog = operator_catalog();
  EXPECT(catalog.size() == 18);
  const OperatorInfo& add = operator_schema(Operator::Add);
  EXPECT(std::string(add.name) == "aten.add" && add.kind == OperatorKind::Binary && add.dtype_rule == DTypeRule::ArithmeticPromotion);
  EXPECT(add.returns_fresh_output());
  EXPECT(add.should_record_autograd(DType::F32, true));
  EXPECT(!add.should_record_autograd(DType::I64, true));
  EXPECT(!add.should_record_autograd(DType::F32, false));
  EXPECT(operator_schema(Operator::Matmul).kind == OperatorKind::MatrixMultiply);
  EXPECT(operator_schema(Operator::Matmul).dtype_rule == DTypeRule::FloatingPromotion);
  EXPECT(operator_schema(Operator::SumDim).kind == OperatorKind::ReductionDim);
  EXPECT(std::string(operator_schema(Operator::LayerNormLastDim).name) == "aten.layer_norm.last_dim");
  EXPECT(operator_schema(Operator::Embedding).dtype_rule == DTypeRule::EmbeddingLookup);
  EXPECT(operator_schema(Operator::MaskedFill).kind == OperatorKind::Masking);
  const OperatorInfo& argmax = operator_schema(Operator::ArgmaxLastDim);
  EXPECT(argmax.autograd_policy == AutogradPolicy::NonDifferentiable && !argmax.should_record_autograd(DType::I64, true));
  EXPECT(std::string(operator_schema(Operator::CausalSelfAttention).name) == "heirloom.causal_self_attention");
  int aten = 0, own = 0;
  for (const auto& s : catalog) {
    if (std::strncmp(s.name, "aten.", 5) == 0) ++aten;
    if (std::strncmp(s.name, "heirloom.", 9) == 0) ++own;
  }
  EXPECT(aten >= 16 && own == 2);

  // tests/custom_ops.rs: names and registry
  EXPECT(throws_with([] { CustomUnaryOp("bad name", square_forward, square_backward); }, "unsupported characters"));
  EXPECT(throws_with([] { CustomUnaryOp("   ", square_forward, square_backward); }, "cannot be empty"));
  EXPECT(throws_with([] { CustomUnaryOp(std::string(129, 'a').c_str(), square_forward, square_backward); }, "at most 128 bytes"));
  CustomUnaryRegistry registry;
  EXPECT(registry.is_empty());
  const CustomUnaryOp square("heirloom.test.square", square_forward, square_backward);
  registry.register_op(square);
  EXPECT(registry.len() == 1 && registry.get("heirloom.test.square").has_value() && !registry.get("missing").has_value());
  EXPECT(throws_with([&] { registry.register_op(square); }, "already registered"));
  const Tensor ints = Tensor::from_i64({1, 2}, {2});
  EXPECT(throws_with([&] { ints.apply_custom_unary(square); }, "floating"));
  // host tensors: forward through the callbacks, dtype preserved, no graph under no_grad
  const Tensor xf = Tensor::from_vec({1.5f, -2.0f}, {2}, true);
  const Tensor yf = xf.apply_custom_unary(square);
  EXPECT(yf.dtype() == DType::F32 && yf.data_f32() == std::vector<float>({2.25f, 4.0f}) && yf.requires_grad());
  const Tensor yn = no_grad([&] { return Tensor::from_f64({2.0}, {1}, true).apply_custom_unary(square); });
  EXPECT(!yn.requires_grad() && yn.data_f64() == std::vector<double>({4.0}));
  EXPECT(throws_with([&] { Tensor::from_f64({2.0, 3.0}, {2}, true).apply_custom_unary(CustomUnaryOp("heirloom.test.bad_forward", bad_forward, square_backward)); },
                     "returned 3 elements"));

  // views are metadata only (src/tensor.rs:2429-2688)
  std::vector<float> vals(24);
  for (int i = 0; i < 24; ++i) vals[i] = (float)i;
  const Tensor t = Tensor::from_vec(vals, {2, 3, 4});
  EXPECT(t.strides() == std::vector<size_t>({12, 4, 1}) && t.is_contiguous() && t.storage_offset() == 0);
  const Tensor tt = t.transpose(0, 2);
  EXPECT(tt.shape() == std::vector<size_t>({4, 3, 2}) && tt.strides() == std::vector<size_t>({1, 4, 12}) && !tt.is_contiguous());
  EXPECT(tt.shares_storage_with(t) && tt.id() != t.id());
  EXPECT(tt.data_f64()[1] == 12.0 && tt.data_f64()[2] == 4.0);
  const Tensor p = t.permute({1, 2, 0});
  EXPECT(p.shape() == std::vector<size_t>({3, 4, 2}) && p.strides() == std::vector<size_t>({4, 1, 12}));
  const Tensor n = t.narrow(1, 1, 2);
  EXPECT(n.shape() == std::vector<size_t>({2, 2, 4}) && n.storage_offset() == 4 && n.data_f64()[0] == 4.0 && n.data_f64()[8] == 16.0);
  const Tensor v = t.view({6, 4});
  EXPECT(v.strides() == std::vector<size_t>({4, 1}) && v.shares_storage_with(t));
  EXPECT(throws_with([&] { tt.view({24}); }, "contiguous"));
  const Tensor r = tt.reshape({24});  // host tensors are copied in logical order
  EXPECT(!r.shares_storage_with(t) && r.data_f64()[1] == 12.0);
  const Tensor e = Tensor::from_vec({1.f, 2.f, 3.f}, {3}).expand({2, 3});
  EXPECT(e.strides() == std::vector<size_t>({0, 1}) && e.data_f64() == std::vector<double>({1, 2, 3, 1, 2, 3}));
  EXPECT(throws_with([&] { t.expand({2, 3, 5}); }, "cannot expand"));
  EXPECT(throws_with([&] { t.narrow(1, 2, 2); }, "exceeds"));
  EXPECT(throws_with([&] { t.view({5, 5}); }, "cannot view"));
  EXPECT(throws_with([&] { t.permute({0, 0, 1}); }, "permutation"));
  EXPECT(throws_with([&] { Tensor::from_vec({1.f}, {2}); }, "does not match shape"));

  // compute is routed to the GPU; a host tensor is refused, never computed on the host
  EXPECT(throws_with([&] { t.gelu(); }, "runs on the GPU only"));
  EXPECT(throws_with([&] { v.matmul(v.transpose(0, 1)); }, "runs on the GPU only"));
  EXPECT(throws_with([&] { t.sum(); }, "runs on the GPU only"));
  // leaves and requires_grad
  Tensor leaf = Tensor::from_vec({1.f, 2.f}, {2});
  EXPECT(leaf.is_leaf() && !leaf.requires_grad() && !leaf.grad().has_value());
  leaf.set_requires_grad(true);
  EXPECT(leaf.requires_grad());
  Tensor il = Tensor::from_i64({1}, {1});
  EXPECT(throws_with([&] { il.set_requires_grad(true); }, "floating"));
  EXPECT(throws_with([&] { leaf.grad_f64(); }, "no gradient"));
}

// ---- GPU -------------------------------------------------------------------------------------------------
static void gpu_tests() {
  const Device dev = Device::cuda(0);
  // tests/custom_ops.rs: chaining and backward on a device tensor (staged through the host)
  {
    const CustomUnaryOp square("heirloom.test.square", square_forward, square_backward);
    const CustomUnaryOp cubic("heirloom.test.shifted_cubic", cubic_forward, cubic_backward);
    const Tensor x = Tensor::from_vec({-2.0f, 0.5f, 3.0f}, {3}, true).to_device(dev);
    const Tensor y = x.apply_custom_unary(square).apply_custom_unary(cubic);
    EXPECT(y.dtype() == DType::F32 && y.device() == dev);
    EXPECT(close(y.data_f64(), {125.0, 1.953125, 1000.0}, 1e-6));
    y.sum().backward();
    EXPECT(close(x.grad_f64(), {-300.0, 4.6875, 1800.0}, 1e-6));
    const CustomUnaryOp bad("heirloom.test.bad_backward", square_forward, bad_backward);
    const Tensor z = Tensor::from_vec({2.0f, 3.0f}, {2}, true).to_device(dev).apply_custom_unary(bad);
    EXPECT(throws_with([&] { z.sum().backward(); }, "returned gradient length"));
  }
  // embedding: repeated indices accumulate (tests/transformer_runtime.rs:1460-1473)
  {
    const Tensor w = Tensor::from_vec({0.f, 0.f, 0.f, 0.f}, {4, 1}, true).to_device(dev);
    const Tensor idx = Tensor::from_i64({0, 1, 0, 1, 2, 3}, {6}).to_device(dev);
    Tensor::embedding(w, idx).sum().backward();
    EXPECT(close(w.grad_f64(), {2, 2, 1, 1}, 1e-7));
  }
  // Linear = x·Wᵀ + b with a transposed view of the weight; gradients arrive contiguous at the leaves
  {
    const Tensor x = Tensor::from_vec({1, 2, 3, 4, 5, 6}, {2, 3}, true).to_device(dev);
    const Tensor w = Tensor::from_vec({1, 0, -1, 0.5f, 0.5f, 0.5f}, {2, 3}, true).to_device(dev);
    const Tensor b = Tensor::from_vec({0.25f, -0.25f}, {2}, true).to_device(dev);
    nn::Linear lin(w, b);
    const Tensor y = lin.forward(x);
    EXPECT(close(y.data_f64(), {-1.75, 2.75, -1.75, 7.25}, 1e-6));
    const Tensor coeff = Tensor::from_vec({1, 2, 3, 4}, {2, 2}).to_device(dev);
    y.mul(coeff).sum().backward();
    EXPECT(close(x.grad_f64(), {2, 1, 0, 5, 2, -1}, 1e-6));           // dY·W
    EXPECT(close(w.grad_f64(), {13, 17, 21, 18, 24, 30}, 1e-6));      // dYᵀ·X
    EXPECT(close(b.grad_f64(), {4, 6}, 1e-6));
    EXPECT(w.grad()->is_contiguous() && w.grad()->shape() == w.shape());
    EXPECT(!y.grad().has_value());  // non-leaf gradients are not kept
  }
  // accumulation by tensor identity: y = x·x + x used twice, and a second backward adds to the leaf
  {
    const Tensor x = Tensor::from_vec({1.5f, -2.0f}, {2}, true).to_device(dev);
    x.mul(x).add(x).sum().backward();
    EXPECT(close(x.grad_f64(), {4.0, -3.0}, 1e-6));
    x.mul(x).sum().backward();
    EXPECT(close(x.grad_f64(), {7.0, -7.0}, 1e-6));
    const Tensor y = no_grad([&] { return x.mul(x); });
    EXPECT(!y.requires_grad());
    EXPECT(throws_with([&] { y.sum().backward(); }, "does not require gradients"));
    EXPECT(throws_with([&] { x.mul(x).backward(); }, "one-element"));
  }
  // narrow and expand backward, mean, relu, softmax rows
  {
    const Tensor x = Tensor::from_vec({1, 2, 3, 4, 5, 6}, {3, 2}, true).to_device(dev);
    x.narrow(0, 1, 2).sum().backward();
    EXPECT(close(x.grad_f64(), {0, 0, 1, 1, 1, 1}, 1e-7));
    const Tensor v = Tensor::from_vec({1, -1}, {2}, true).to_device(dev);
    // a stride-0 view is consumable by matmul (the one device op that takes strided operands)
    v.expand({3, 2}).matmul(Tensor::from_vec({1, 2}, {2, 1}).to_device(dev)).sum().backward();
    EXPECT(close(v.grad_f64(), {3, 6}, 1e-6));
    const Tensor r = Tensor::from_vec({-1, 2, -3, 4}, {4}, true).to_device(dev);
    r.relu().mean().backward();
    EXPECT(close(r.grad_f64(), {0, 0.25, 0, 0.25}, 1e-7));
    const Tensor s = Tensor::from_vec({0, 0, 0, 0}, {2, 2}, true).to_device(dev);
    const Tensor pr = s.softmax_dim(1);
    EXPECT(close(pr.data_f64(), {0.5, 0.5, 0.5, 0.5}, 1e-7));
    pr.mul(Tensor::from_vec({1, 0, 0, 1}, {2, 2}).to_device(dev)).sum().backward();
    EXPECT(close(s.grad_f64(), {0.25, -0.25, -0.25, 0.25}, 1e-6));
  }
  // device kernels demand contiguous inputs; matmul alone takes strided views
  {
    const Tensor x = Tensor::from_vec({1, 2, 3, 4, 5, 6}, {2, 3}).to_device(dev);
    EXPECT(throws_with([&] { x.transpose(0, 1).gelu(); }, "contiguous"));
    EXPECT(close(x.matmul(x.transpose(0, 1)).data_f64(), {14, 32, 32, 77}, 1e-6));
    EXPECT(throws_with([&] { x.matmul(x); }, "inner dimensions"));
    EXPECT(throws_with([&] { x.add(Tensor::from_vec({1, 2}, {2})); }, "different devices"));
  }
  // AdamW: one step against the closed form; parameters without a gradient are skipped, the step
  // counter advances once per call (src/nn.rs:2156-2220)
  {
    Tensor p = Tensor::from_vec({1.0f, -2.0f}, {2}, true).to_device(dev);
    Tensor q = Tensor::from_vec({3.0f}, {1}, true).to_device(dev);
    nn::AdamW opt({p, q}, 0.05, 0.9, 0.999, 1e-8, 0.01);
    p.mul(p).sum().backward();  // g = 2p
    opt.step();
    std::vector<double> want;
    for (double pv : {1.0, -2.0}) {
      const double g = 2.0 * pv + 0.01 * pv, m = 0.1 * g, v = 0.001 * g * g;
      want.push_back(pv - 0.05 * (m / 0.1) / (std::sqrt(v / 0.001) + 1e-8));
    }
    EXPECT(close(p.data_f64(), want, 1e-6));
    EXPECT(close(q.data_f64(), {3.0}, 0.0) && opt.step_count() == 1 && p.storage_version() == 1 && q.storage_version() == 0);
    opt.zero_grad();
    EXPECT(!p.grad().has_value());
    opt.step();
    EXPECT(opt.step_count() == 2 && close(p.data_f64(), want, 1e-6));
  }
  const RuntimeCounters c = cuda_runtime_counters(0);
  EXPECT(c.launches > 20);
}

// ---- one decoder training step from the nn modules --------------------------------------------------------
struct Reader {
  std::ifstream in;
  explicit Reader(const char* path) : in(path, std::ios::binary) {
    if (!in) throw std::runtime_error(std::string("cannot open ") + path);
  }
  int64_t i64() { int64_t v; in.read(reinterpret_cast<char*>(&v), 8); return v; }
  std::vector<float> floats(size_t n) { std::vector<float> v(n); in.read(reinterpret_cast<char*>(v.data()), n * 4); return v; }
  std::vector<int64_t> ints(size_t n) { std::vector<int64_t> v(n); in.read(reinterpret_cast<char*>(v.data()), n * 8); return v; }
};

static int decoder_step(const char* in_path, const char* out_path) {
  Reader rd(in_path);
  const size_t V = rd.i64(), d = rd.i64(), L = rd.i64(), H = rd.i64(), F = rd.i64(), ctx_len = rd.i64(), B = rd.i64(), T = rd.i64();
  const Device dev = Device::cuda(0);
  std::vector<Tensor> params;  // state-dict order (src/memory_transformer.rs:2098-2117)
  auto param = [&](const std::vector<size_t>& shape) {
    size_t n = 1;
    for (size_t s : shape) n *= s;
    Tensor t = Tensor::from_vec(rd.floats(n), shape, true).to_device(dev);
    params.push_back(t);
    return t;
  };
  nn::Embedding tok{param({V, d})}, pos{param({ctx_len, d})};
  std::vector<nn::TransformerBlock> blocks(L);
  for (auto& b : blocks) {
    b.ln1.weight = param({d}); b.ln1.bias = param({d});
    for (nn::Linear* lin : {&b.attention.q_proj, &b.attention.k_proj, &b.attention.v_proj, &b.attention.out_proj}) {
      lin->weight = param({d, d});
      lin->bias = param({d});
    }
    b.attention.n_heads = H;
    b.ln2.weight = param({d}); b.ln2.bias = param({d});
    b.feed_forward.fc1.weight = param({F, d}); b.feed_forward.fc1.bias = param({F});
    b.feed_forward.fc2.weight = param({d, F}); b.feed_forward.fc2.bias = param({d});
  }
  nn::LayerNorm ln_f;
  ln_f.weight = param({d}); ln_f.bias = param({d});
  nn::Linear lm_head;
  lm_head.weight = param({V, d}); lm_head.bias = param({V});
  const std::vector<int64_t> tokens = rd.ints(B * T), targets = rd.ints(B * T);
  std::vector<int64_t> positions(B * T);
  for (size_t i = 0; i < B * T; ++i) positions[i] = (int64_t)(i % T);

  nn::AdamW opt(params, 1e-3, 0.9, 0.999, 1e-8, 0.01);
  opt.zero_grad();
  // MemoryTransformerLm::forward (src/memory_transformer.rs:2069-2081) and loss (:1604-1610)
  Tensor x = tok.forward(Tensor::from_i64(tokens, {B, T}).to_device(dev))
                 .add(pos.forward(Tensor::from_i64(positions, {B, T}).to_device(dev)))
                 .reshape({B * T, d});
  for (const auto& b : blocks) x = b.forward(x, B, T);
  const Tensor logits = lm_head.forward(ln_f.forward(x));
  const Tensor loss = logits.cross_entropy_for_logits(Tensor::from_i64(targets, {B * T}).to_device(dev));
  loss.backward();

  std::ofstream out(out_path, std::ios::binary);
  const float loss_value = (float)loss.item();
  out.write(reinterpret_cast<const char*>(&loss_value), 4);
  for (const auto& p : params) {
    const std::vector<float> g = p.grad().value().data_f32();
    out.write(reinterpret_cast<const char*>(g.data()), g.size() * 4);
  }
  opt.step();
  for (const auto& p : params) {
    const std::vector<float> v = p.data_f32();
    out.write(reinterpret_cast<const char*>(v.data()), v.size() * 4);
  }
  return out.good() ? 0 : 1;
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "";
  try {
    if (mode == "cpu") cpu_tests();
    else if (mode == "gpu") gpu_tests();
    else if (mode == "decoder" && argc == 4) return decoder_step(argv[2], argv[3]);
    else {
      std::printf("usage: host_tests cpu | gpu | decoder IN OUT\n");
      return 2;
    }
  } catch (const std::exception& e) {
    std::printf("FAIL: unexpected exception: %s\n", e.what());
    return 1;
  }
  std::printf("%s: %d failure(s)\n", mode.c_str(), g_failures);
  return g_failures == 0 ? 0 : 1;
}
