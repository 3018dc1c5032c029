// CPU restatement of the reference's training step for the dense decoder, in C++.
//
// TEST INFRASTRUCTURE, not product code: only the tests, the smoke check and the benchmark's CPU
// legs may load this library.  It restates, op by op, what the reference's CPU path computes:
// every op reads its inputs as f64, computes in f64 and rounds its output to f32
// (src/tensor.rs:5179-5191); gradients stay f64 through the whole backward and reach AdamW as f64
// (src/nn.rs:2441-2453); the backward of matmul is the reference's scalar triple loop in its own
// loop order (src/tensor/autograd.rs:2085-2099).  The forward matmul of the reference goes through
// the `matrixmultiply` crate (0.3.10, not vendored); a plain f64 loop stands in for it here (the
// summation order differs by a few ulp of f64, far below the f32 rounding of the output).
// Single-threaded, as the reference is for rank-2 operands.
//
// Parity of this file is pinned two ways: against the NumPy oracle (same ops, independent code) and,
// through it, against the reference's own fixtures.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

typedef std::vector<double> Vec;

inline double f32r(double x) { return (double)(float)x; }

// f32 -> bf16 -> f32, round to nearest even, NaN quieted (src/storage.rs:440-449, src/nn.rs:250-261)
inline double bf16r(double x) {
  float f = (float)x;
  uint32_t bits;
  std::memcpy(&bits, &f, 4);
  uint32_t out;
  if (f != f) out = ((bits >> 16) | 0x0040u) << 16;
  else out = ((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16) << 16;
  std::memcpy(&f, &out, 4);
  return (double)f;
}

struct Config { int vocab, d_model, n_layers, n_heads, d_ff, context; };

// state-dict order (src/memory_transformer.rs:2098-2117)
struct Layout {
  size_t tok, pos;
  struct Block { size_t ln1_w, ln1_b, q_w, q_b, k_w, k_b, v_w, v_b, o_w, o_b, ln2_w, ln2_b, fc1_w, fc1_b, fc2_w, fc2_b; };
  std::vector<Block> blocks;
  size_t lnf_w, lnf_b, head_w, head_b, total;
};

Layout make_layout(const Config& c) {
  Layout l;
  size_t at = 0;
  auto take = [&](size_t n) { size_t o = at; at += n; return o; };
  const size_t d = c.d_model, f = c.d_ff;
  l.tok = take((size_t)c.vocab * d);
  l.pos = take((size_t)c.context * d);
  for (int i = 0; i < c.n_layers; ++i) {
    Layout::Block b;
    b.ln1_w = take(d); b.ln1_b = take(d);
    b.q_w = take(d * d); b.q_b = take(d);
    b.k_w = take(d * d); b.k_b = take(d);
    b.v_w = take(d * d); b.v_b = take(d);
    b.o_w = take(d * d); b.o_b = take(d);
    b.ln2_w = take(d); b.ln2_b = take(d);
    b.fc1_w = take(f * d); b.fc1_b = take(f);
    b.fc2_w = take(d * f); b.fc2_b = take(d);
    l.blocks.push_back(b);
  }
  l.lnf_w = take(d); l.lnf_b = take(d);
  l.head_w = take((size_t)c.vocab * d); l.head_b = take(c.vocab);
  l.total = at;
  return l;
}

// ---- ops -------------------------------------------------------------------------------------------

// Embedding::forward (src/tensor.rs:3337-3395)
void embedding(const double* w, const int64_t* idx, size_t n, size_t dim, Vec& out) {
  out.resize(n * dim);
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j < dim; ++j) out[i * dim + j] = f32r(w[(size_t)idx[i] * dim + j]);
}
// scatter-add, repeats accumulate (src/tensor/autograd.rs:2234-2261)
void embedding_backward(const int64_t* idx, size_t n, size_t dim, const double* gout, double* gw) {
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j < dim; ++j) gw[(size_t)idx[i] * dim + j] += gout[i * dim + j];
}

// LayerNorm (src/tensor.rs:3175-3256): biased variance, rstd = 1/sqrt(var + eps)
void layer_norm(const Vec& x, const double* w, const double* b, size_t rows, size_t feat, Vec& out) {
  out.resize(rows * feat);
  for (size_t r = 0; r < rows; ++r) {
    const double* xr = &x[r * feat];
    double mean = 0.0;
    for (size_t j = 0; j < feat; ++j) mean += xr[j];
    mean /= (double)feat;
    double var = 0.0;
    for (size_t j = 0; j < feat; ++j) { const double d = xr[j] - mean; var += d * d; }
    var /= (double)feat;
    const double rstd = 1.0 / std::sqrt(var + 1e-5);
    for (size_t j = 0; j < feat; ++j) out[r * feat + j] = f32r((xr[j] - mean) * rstd * w[j] + b[j]);
  }
}
// src/tensor/autograd.rs:2158-2232
void layer_norm_backward(const Vec& x, const double* w, const Vec& g, size_t rows, size_t feat, Vec& dx, double* dw,
                         double* db) {
  dx.resize(rows * feat);
  std::vector<double> xhat(feat), dxhat(feat);
  for (size_t r = 0; r < rows; ++r) {
    const double* xr = &x[r * feat];
    const double* gr = &g[r * feat];
    double mean = 0.0;
    for (size_t j = 0; j < feat; ++j) mean += xr[j];
    mean /= (double)feat;
    double var = 0.0;
    for (size_t j = 0; j < feat; ++j) { const double d = xr[j] - mean; var += d * d; }
    var /= (double)feat;
    const double rstd = 1.0 / std::sqrt(var + 1e-5);
    double s1 = 0.0, s2 = 0.0;
    for (size_t j = 0; j < feat; ++j) {
      xhat[j] = (xr[j] - mean) * rstd;
      dxhat[j] = gr[j] * w[j];
      s1 += dxhat[j];
      s2 += dxhat[j] * xhat[j];
      dw[j] += gr[j] * xhat[j];
      db[j] += gr[j];
    }
    for (size_t j = 0; j < feat; ++j)
      dx[r * feat + j] = rstd * ((double)feat * dxhat[j] - s1 - xhat[j] * s2) / (double)feat;
  }
}

// Linear::forward = x·Wᵀ + b (src/nn.rs:454-475); W is [out, in].  Under AMP both operands are rounded
// to bf16 and the f32 product gets the f32 bias (src/nn.rs:338-450).
void linear(const Vec& x, const double* w, const double* b, size_t rows, size_t in, size_t out_f, bool amp, Vec& y) {
  y.assign(rows * out_f, 0.0);
  Vec xa, wa;
  const double* xp = x.data();
  const double* wp = w;
  if (amp) {
    xa.resize(rows * in);
    for (size_t i = 0; i < rows * in; ++i) xa[i] = bf16r(x[i]);
    wa.resize(out_f * in);
    for (size_t i = 0; i < out_f * in; ++i) wa[i] = bf16r(w[i]);
    xp = xa.data();
    wp = wa.data();
  }
  for (size_t r = 0; r < rows; ++r)
    for (size_t o = 0; o < out_f; ++o) {
      double acc = 0.0;
      const double* xr = xp + r * in;
      const double* wr = wp + o * in;
      for (size_t k = 0; k < in; ++k) acc += xr[k] * wr[k];
      y[r * out_f + o] = f32r(f32r(acc) + b[o]);
    }
}
// dX = dY·W, dW = dYᵀ·X, db = Σ dY.  The loop nest is the reference's: rows, then the shared
// dimension, then output columns, accumulating both gradients in the innermost statement
// (src/tensor/autograd.rs:2085-2099, with left = x [rows, in] and right = Wᵀ [in, out]).
void linear_backward(const Vec& x, const double* w, const Vec& gy, size_t rows, size_t in, size_t out_f, bool amp,
                     Vec& dx, double* dw, double* db) {
  dx.assign(rows * in, 0.0);
  Vec xa, wa, ga;
  const double* xp = x.data();
  const double* wp = w;
  const double* gp = gy.data();
  for (size_t r = 0; r < rows; ++r)
    for (size_t o = 0; o < out_f; ++o) db[o] += gy[r * out_f + o];
  if (amp) {  // dY, X and W enter the products as bf16 operands (src/tensor/autograd.rs:795-850)
    xa.resize(rows * in);
    for (size_t i = 0; i < rows * in; ++i) xa[i] = bf16r(x[i]);
    wa.resize(out_f * in);
    for (size_t i = 0; i < out_f * in; ++i) wa[i] = bf16r(w[i]);
    ga.resize(rows * out_f);
    for (size_t i = 0; i < rows * out_f; ++i) ga[i] = bf16r(gy[i]);
    xp = xa.data(); wp = wa.data(); gp = ga.data();
  }
  Vec dwt((size_t)in * out_f, 0.0);  // gradient of the transposed view [in, out]
  for (size_t r = 0; r < rows; ++r)
    for (size_t s = 0; s < in; ++s) {
      const double left = xp[r * in + s];
      double acc = 0.0;
      double* dwrow = &dwt[s * out_f];
      const double* grow = gp + r * out_f;
      for (size_t c = 0; c < out_f; ++c) {
        const double go = grow[c];
        acc += go * wp[c * in + s];  // right[s, c] = W[c, s]
        dwrow[c] += left * go;
      }
      dx[r * in + s] += acc;
    }
  for (size_t s = 0; s < in; ++s)
    for (size_t c = 0; c < out_f; ++c) dw[c * in + s] += dwt[s * out_f + c];
  if (amp) {  // the CUDA route stores each product as an f32 tensor
    for (size_t i = 0; i < rows * in; ++i) dx[i] = f32r(dx[i]);
  }
}

const double kGeluC = 0.7978845608028654;  // sqrt(2/pi)
// src/tensor.rs:5152-5154
inline double gelu_value(double x) { return 0.5 * x * (1.0 + std::tanh(kGeluC * (x + 0.044715 * x * x * x))); }
// src/tensor/autograd.rs:2891-2897
inline double gelu_grad(double x) {
  const double t = std::tanh(kGeluC * (x + 0.044715 * x * x * x));
  return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * kGeluC * (1.0 + 3.0 * 0.044715 * x * x);
}

// Tensor::causal_self_attention (src/tensor.rs:3980-4098); heads interleaved along the channel
// dimension (index = b·T·C + t·C + h·hd + j, src/tensor.rs:5156-5177).  Saves P [B,H,T,T].
void attention(const Vec& q, const Vec& k, const Vec& v, int B, int T, int C, int H, bool amp, Vec& out, Vec& probs) {
  const int hd = C / H;
  const double scale = 1.0 / std::sqrt((double)hd);
  out.assign((size_t)B * T * C, 0.0);
  probs.assign((size_t)B * H * T * T, 0.0);
  std::vector<double> s(T);
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < H; ++h)
      for (int t = 0; t < T; ++t) {
        const double* qr = &q[((size_t)b * T + t) * C + h * hd];
        double m = -INFINITY;
        for (int u = 0; u <= t; ++u) {
          const double* kr = &k[((size_t)b * T + u) * C + h * hd];
          double acc = 0.0;
          for (int j = 0; j < hd; ++j) acc += qr[j] * kr[j];
          s[u] = acc * scale;
          m = std::max(m, s[u]);
        }
        double sum = 0.0;
        for (int u = 0; u <= t; ++u) { s[u] = std::exp(s[u] - m); sum += s[u]; }
        double* pr = &probs[(((size_t)b * H + h) * T + t) * T];
        double* orow = &out[((size_t)b * T + t) * C + h * hd];
        for (int u = 0; u <= t; ++u) {
          pr[u] = s[u] / sum;
          const double pu = amp ? bf16r(pr[u]) : pr[u];  // P is a bf16 operand on the tensor-core route
          const double* vr = &v[((size_t)b * T + u) * C + h * hd];
          for (int j = 0; j < hd; ++j) orow[j] += pu * vr[j];
        }
        for (int j = 0; j < hd; ++j) orow[j] = f32r(orow[j]);
      }
}
// dQ, dK, dV from the saved P (src/tensor/autograd.rs:2623-2712); with AMP the products take
// bf16-rounded dO, P and dS operands (src/tensor/autograd.rs:1626-1914).
void attention_backward(const Vec& q, const Vec& k, const Vec& v, const Vec& probs, const Vec& go_in, int B, int T, int C,
                        int H, bool amp, Vec& dq, Vec& dk, Vec& dv) {
  const int hd = C / H;
  const double scale = 1.0 / std::sqrt((double)hd);
  dq.assign((size_t)B * T * C, 0.0);
  dk.assign((size_t)B * T * C, 0.0);
  dv.assign((size_t)B * T * C, 0.0);
  std::vector<double> dp(T), gor(hd);
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < H; ++h)
      for (int t = 0; t < T; ++t) {
        const size_t row = ((size_t)b * T + t) * C + h * hd;
        for (int j = 0; j < hd; ++j) gor[j] = amp ? bf16r(go_in[row + j]) : go_in[row + j];
        const double* pr = &probs[(((size_t)b * H + h) * T + t) * T];
        double dot = 0.0;
        for (int u = 0; u <= t; ++u) {
          const size_t col = ((size_t)b * T + u) * C + h * hd;
          const double pu = amp ? bf16r(pr[u]) : pr[u];
          double acc = 0.0;
          for (int j = 0; j < hd; ++j) {
            dv[col + j] += pu * gor[j];
            acc += gor[j] * v[col + j];
          }
          dp[u] = acc;
          dot += acc * pr[u];
        }
        for (int u = 0; u <= t; ++u) {
          const size_t col = ((size_t)b * T + u) * C + h * hd;
          double ds = pr[u] * (dp[u] - dot) * scale;
          if (amp) ds = bf16r(ds);
          for (int j = 0; j < hd; ++j) {
            dq[row + j] += ds * k[col + j];
            dk[col + j] += ds * q[row + j];
          }
        }
      }
}

// mean over rows of −z[y] + max + ln Σ exp(z − max) (src/tensor.rs:4816-4882) and
// dz = (softmax − onehot)/N (src/tensor/autograd.rs:2591-2621)
double cross_entropy(const Vec& z, const int64_t* targets, size_t rows, size_t classes, Vec& dz) {
  dz.resize(rows * classes);
  double total = 0.0;
  for (size_t r = 0; r < rows; ++r) {
    const double* zr = &z[r * classes];
    double m = -INFINITY;
    for (size_t c = 0; c < classes; ++c) m = std::max(m, zr[c]);
    double sum = 0.0;
    for (size_t c = 0; c < classes; ++c) sum += std::exp(zr[c] - m);
    total += -zr[targets[r]] + m + std::log(sum);
    for (size_t c = 0; c < classes; ++c) dz[r * classes + c] = std::exp(zr[c] - m) / sum;
    dz[r * classes + targets[r]] -= 1.0;
    for (size_t c = 0; c < classes; ++c) dz[r * classes + c] *= 1.0 / (double)rows;
  }
  return f32r(total / (double)rows);
}

struct Saved { Vec x, a, q, k, v, probs, o, r, c, h, g; };

// MemoryTransformerLm::forward + loss + backward for the dense decoder
// (src/memory_transformer.rs:2069-2081, :1604-1610; block :1176-1183; AMP round trips :1636-1662,
// :1153-1172, src/nn.rs:718-788, :873-884).
double loss_and_grads(const Config& cfg, const double* p, const int64_t* tokens, const int64_t* targets, int B, int T,
                      bool amp, bool grad_f32, double* grads) {
  const Layout L = make_layout(cfg);
  const size_t N = (size_t)B * T, d = cfg.d_model, F = cfg.d_ff, V = cfg.vocab;
  const int H = cfg.n_heads;
  auto rt = [&](Vec& a) { if (amp) for (auto& e : a) e = bf16r(e); };
  auto gr = [&](Vec& a) { if (amp || grad_f32) for (auto& e : a) e = f32r(e); };
  std::fill(grads, grads + L.total, 0.0);

  std::vector<int64_t> pos_ids(N);
  for (size_t i = 0; i < N; ++i) pos_ids[i] = (int64_t)(i % T);
  Vec tok, pos, x(N * d);
  embedding(p + L.tok, tokens, N, d, tok); rt(tok);
  embedding(p + L.pos, pos_ids.data(), N, d, pos); rt(pos);
  for (size_t i = 0; i < N * d; ++i) x[i] = f32r(tok[i] + pos[i]);
  rt(x);
  std::vector<Saved> saved(cfg.n_layers);
  for (int i = 0; i < cfg.n_layers; ++i) {
    const Layout::Block& b = L.blocks[i];
    Saved& s = saved[i];
    s.x = x;
    layer_norm(x, p + b.ln1_w, p + b.ln1_b, N, d, s.a); rt(s.a);
    linear(s.a, p + b.q_w, p + b.q_b, N, d, d, amp, s.q); rt(s.q);
    linear(s.a, p + b.k_w, p + b.k_b, N, d, d, amp, s.k); rt(s.k);
    linear(s.a, p + b.v_w, p + b.v_b, N, d, d, amp, s.v); rt(s.v);
    attention(s.q, s.k, s.v, B, T, (int)d, H, amp, s.o, s.probs); rt(s.o);
    Vec pr;
    linear(s.o, p + b.o_w, p + b.o_b, N, d, d, amp, pr); rt(pr);
    s.r.resize(N * d);
    for (size_t j = 0; j < N * d; ++j) s.r[j] = f32r(x[j] + pr[j]);
    rt(s.r);
    layer_norm(s.r, p + b.ln2_w, p + b.ln2_b, N, d, s.c); rt(s.c);
    linear(s.c, p + b.fc1_w, p + b.fc1_b, N, d, F, amp, s.h); rt(s.h);
    s.g.resize(N * F);
    for (size_t j = 0; j < N * F; ++j) s.g[j] = f32r(gelu_value(s.h[j]));
    rt(s.g);
    Vec f;
    linear(s.g, p + b.fc2_w, p + b.fc2_b, N, F, d, amp, f); rt(f);
    for (size_t j = 0; j < N * d; ++j) x[j] = f32r(s.r[j] + f[j]);
    rt(x);
  }
  Vec z, logits, dlogits;
  layer_norm(x, p + L.lnf_w, p + L.lnf_b, N, d, z); rt(z);
  linear(z, p + L.head_w, p + L.head_b, N, d, V, amp, logits);
  const double loss = cross_entropy(logits, targets, N, V, dlogits);
  gr(dlogits);

  Vec dz, dx, tmp;
  linear_backward(z, p + L.head_w, dlogits, N, d, V, amp, dz, grads + L.head_w, grads + L.head_b);
  gr(dz);
  layer_norm_backward(x, p + L.lnf_w, dz, N, d, dx, grads + L.lnf_w, grads + L.lnf_b);
  gr(dx);
  for (int i = cfg.n_layers - 1; i >= 0; --i) {
    const Layout::Block& b = L.blocks[i];
    Saved& s = saved[i];
    Vec dg, dh(N * F), dc, dr_ln, dr(N * d), dO, dq, dk, dv, da(N * d, 0.0), dai, dx_ln;
    linear_backward(s.g, p + b.fc2_w, dx, N, F, d, amp, dg, grads + b.fc2_w, grads + b.fc2_b);
    gr(dg);
    for (size_t j = 0; j < N * F; ++j) dh[j] = dg[j] * gelu_grad(s.h[j]);
    gr(dh);
    linear_backward(s.c, p + b.fc1_w, dh, N, d, F, amp, dc, grads + b.fc1_w, grads + b.fc1_b);
    gr(dc);
    layer_norm_backward(s.r, p + b.ln2_w, dc, N, d, dr_ln, grads + b.ln2_w, grads + b.ln2_b);
    gr(dr_ln);
    for (size_t j = 0; j < N * d; ++j) dr[j] = dx[j] + dr_ln[j];
    gr(dr);
    linear_backward(s.o, p + b.o_w, dr, N, d, d, amp, dO, grads + b.o_w, grads + b.o_b);
    gr(dO);
    attention_backward(s.q, s.k, s.v, s.probs, dO, B, T, (int)d, H, amp, dq, dk, dv);
    gr(dq); gr(dk); gr(dv);
    const size_t w_off[3] = {b.q_w, b.k_w, b.v_w}, b_off[3] = {b.q_b, b.k_b, b.v_b};
    Vec* dproj[3] = {&dq, &dk, &dv};
    for (int j = 0; j < 3; ++j) {
      linear_backward(s.a, p + w_off[j], *dproj[j], N, d, d, amp, dai, grads + w_off[j], grads + b_off[j]);
      for (size_t e = 0; e < N * d; ++e) da[e] += dai[e];
      gr(da);
    }
    layer_norm_backward(s.x, p + b.ln1_w, da, N, d, dx_ln, grads + b.ln1_w, grads + b.ln1_b);
    gr(dx_ln);
    for (size_t j = 0; j < N * d; ++j) dx[j] = dr[j] + dx_ln[j];
    gr(dx);
  }
  embedding_backward(tokens, N, d, dx.data(), grads + L.tok);
  embedding_backward(pos_ids.data(), N, d, dx.data(), grads + L.pos);
  if (amp || grad_f32)
    for (size_t i = 0; i < L.total; ++i) grads[i] = f32r(grads[i]);
  return loss;
}

}  // namespace

extern "C" {

struct hr_config { int vocab, d_model, n_layers, n_heads, d_ff, context; };

// Number of parameter elements in state-dict order.
long long hr_param_count(const hr_config* c) {
  Config cfg{c->vocab, c->d_model, c->n_layers, c->n_heads, c->d_ff, c->context};
  return (long long)make_layout(cfg).total;
}

// Loss and flat f64 gradients of one batch; tokens and targets are [B, T] i64.
double hr_loss_and_grads(const hr_config* c, const double* params, const int64_t* tokens, const int64_t* targets, int B,
                         int T, int amp, int grad_f32, double* grads) {
  Config cfg{c->vocab, c->d_model, c->n_layers, c->n_heads, c->d_ff, c->context};
  return loss_and_grads(cfg, params, tokens, targets, B, T, amp != 0, grad_f32 != 0, grads);
}

// One coupled-decay AdamW step over a flat parameter vector: f64 moments, parameters rounded to f32
// (src/nn.rs:2156-2220, body :2433-2465, clip :2589-2665).  `step` is the value after the increment;
// clip_norm < 0 means none.
void hr_adamw_step(double* params, const double* grads, double* m, double* v, long long n, int step, double lr,
                   double beta1, double beta2, double eps, double wd, double clip_norm) {
  double clip = 1.0;
  if (clip_norm >= 0.0) {
    double ss = 0.0;
    for (long long i = 0; i < n; ++i) ss += grads[i] * grads[i];
    const double norm = std::sqrt(ss);
    if (norm > clip_norm) clip = clip_norm / (norm + 1e-12);
  }
  const double bias1 = 1.0 - std::pow(beta1, step), bias2 = 1.0 - std::pow(beta2, step);
  for (long long i = 0; i < n; ++i) {
    const double g = grads[i] * clip + wd * params[i];
    m[i] = beta1 * m[i] + (1.0 - beta1) * g;
    v[i] = beta2 * v[i] + (1.0 - beta2) * g * g;
    params[i] = f32r(params[i] - lr * (m[i] / bias1) / (std::sqrt(v[i] / bias2) + eps));
  }
}

// zero_grad -> loss -> backward -> AdamW.step for `steps` batches
// (src/bin/heirloom/commands/training.rs:125-167).  tokens_all is [steps][B][T+1]; inputs are its
// first T columns and targets the last T.  m, v start wherever the caller left them; first_step is
// the optimizer's step counter before the first batch.
void hr_train_steps(const hr_config* c, double* params, double* m, double* v, const int64_t* tokens_all, int steps, int B,
                    int T, int first_step, double lr, double beta1, double beta2, double eps, double wd, double clip_norm,
                    int amp, int grad_f32, double* losses) {
  Config cfg{c->vocab, c->d_model, c->n_layers, c->n_heads, c->d_ff, c->context};
  const size_t total = make_layout(cfg).total;
  Vec grads(total);
  std::vector<int64_t> tok((size_t)B * T), tgt((size_t)B * T);
  for (int s = 0; s < steps; ++s) {
    const int64_t* batch = tokens_all + (size_t)s * B * (T + 1);
    for (int b = 0; b < B; ++b)
      for (int t = 0; t < T; ++t) {
        tok[(size_t)b * T + t] = batch[(size_t)b * (T + 1) + t];
        tgt[(size_t)b * T + t] = batch[(size_t)b * (T + 1) + t + 1];
      }
    losses[s] = loss_and_grads(cfg, params, tok.data(), tgt.data(), B, T, amp != 0, grad_f32 != 0, grads.data());
    hr_adamw_step(params, grads.data(), m, v, (long long)total, first_step + s + 1, lr, beta1, beta2, eps, wd, clip_norm);
  }
}

}  // extern "C"
