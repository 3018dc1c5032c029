// f32 kernels with f64 accumulation for the f32 parity route: strided matmul and causal
// attention with materialised probabilities.  These follow the reference's f32 CUDA entries
// (heirloom-kernels/src/ptx/kernels.ptx:1290-1659 matmul, :3760-4609 attention) in what they
// compute, but accumulate in double so that their f32 results round from the same f64 values
// the reference's CPU path produces (src/tensor.rs:577-590).  Not a throughput path.
#include "common.cuh"

namespace hl {
namespace {

constexpr int MT = 16;

__global__ void matmul_f32_strided_kernel(const float* __restrict__ a, hl_matrix_layout la, const float* __restrict__ b,
                                          hl_matrix_layout lb, float* __restrict__ out, hl_matrix_layout lo,
                                          int accumulate) {
  __shared__ double sa[MT][MT + 1];
  __shared__ double sb[MT][MT + 1];
  const long long row = blockIdx.y * (long long)MT + threadIdx.y;
  const long long col = blockIdx.x * (long long)MT + threadIdx.x;
  const long long K = la.cols;
  double acc = 0.0;
  for (long long k0 = 0; k0 < K; k0 += MT) {
    const long long ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
    sa[threadIdx.y][threadIdx.x] =
        (row < la.rows && ka < K) ? (double)a[la.offset + row * la.row_stride + ka * la.col_stride] : 0.0;
    sb[threadIdx.y][threadIdx.x] =
        (kb < K && col < lb.cols) ? (double)b[lb.offset + kb * lb.row_stride + col * lb.col_stride] : 0.0;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MT; ++k) acc += sa[threadIdx.y][k] * sb[k][threadIdx.x];
    __syncthreads();
  }
  if (row < lo.rows && col < lo.cols) {
    float* dst = out + lo.offset + row * lo.row_stride + col * lo.col_stride;
    *dst = accumulate ? (float)((double)*dst + acc) : (float)acc;
  }
}

// q,k,v,out: [B,T,C], heads interleaved along C (index b*T*C + t*C + h*hd + j, as
// src/tensor.rs:5156-5177).  probs: [B,H,T,T] (only s <= t is written; the rest is zeroed).
__global__ void attention_f32_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                         const float* __restrict__ v, float* __restrict__ out, float* __restrict__ probs,
                                         int B, int T, int C, int H) {
  const int hd = C / H;
  const int lane = threadIdx.x & 31;
  const long long w = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)B * H * T) return;
  const int t = (int)(w % T);
  const int h = (int)((w / T) % H);
  const int b = (int)(w / ((long long)T * H));
  const double scale = 1.0 / sqrt((double)hd);
  const float* qr = q + ((size_t)b * T + t) * C + (size_t)h * hd;
  float* pr = probs + (((size_t)b * H + h) * T + t) * (size_t)T;
  double mx = -INFINITY;
  for (int s = lane; s <= t; s += 32) {
    const float* kr = k + ((size_t)b * T + s) * C + (size_t)h * hd;
    double dot = 0.0;
    for (int j = 0; j < hd; ++j) dot += (double)qr[j] * (double)kr[j];
    dot *= scale;
    mx = max(mx, dot);
  }
  mx = warp_max(mx);
  __syncwarp();
  double denom = 0.0;
  for (int s = lane; s <= t; s += 32) {
    const float* kr = k + ((size_t)b * T + s) * C + (size_t)h * hd;
    double dot = 0.0;
    for (int j = 0; j < hd; ++j) dot += (double)qr[j] * (double)kr[j];
    denom += exp(dot * scale - mx);
  }
  denom = warp_sum(denom);
  for (int s = lane; s < T; s += 32) {
    if (s <= t) {
      const float* kr = k + ((size_t)b * T + s) * C + (size_t)h * hd;
      double dot = 0.0;
      for (int j = 0; j < hd; ++j) dot += (double)qr[j] * (double)kr[j];
      pr[s] = (float)(exp(dot * scale - mx) / denom);
    } else {
      pr[s] = 0.f;
    }
  }
  __syncwarp();
  float* orow = out + ((size_t)b * T + t) * C + (size_t)h * hd;
  for (int j = lane; j < hd; j += 32) {
    double acc = 0.0;
    for (int s = 0; s <= t; ++s) acc += (double)pr[s] * (double)v[((size_t)b * T + s) * C + (size_t)h * hd + j];
    orow[j] = (float)acc;
  }
}

// Per query row: dP, dS (written to ds scratch) and dQ.
__global__ void attention_f32_bwd_rows_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                              const float* __restrict__ probs, const float* __restrict__ dout,
                                              float* __restrict__ ds, float* __restrict__ dq, int B, int T, int C, int H) {
  const int hd = C / H;
  const int lane = threadIdx.x & 31;
  const long long w = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)B * H * T) return;
  const int t = (int)(w % T);
  const int h = (int)((w / T) % H);
  const int b = (int)(w / ((long long)T * H));
  const double scale = 1.0 / sqrt((double)hd);
  const float* pr = probs + (((size_t)b * H + h) * T + t) * (size_t)T;
  float* dsr = ds + (((size_t)b * H + h) * T + t) * (size_t)T;
  const float* gor = dout + ((size_t)b * T + t) * C + (size_t)h * hd;
  double dot_sum = 0.0;
  for (int s = lane; s <= t; s += 32) {
    const float* vr = v + ((size_t)b * T + s) * C + (size_t)h * hd;
    double dp = 0.0;
    for (int j = 0; j < hd; ++j) dp += (double)gor[j] * (double)vr[j];
    dot_sum += dp * (double)pr[s];
  }
  dot_sum = warp_sum(dot_sum);
  for (int s = lane; s < T; s += 32) {
    if (s <= t) {
      const float* vr = v + ((size_t)b * T + s) * C + (size_t)h * hd;
      double dp = 0.0;
      for (int j = 0; j < hd; ++j) dp += (double)gor[j] * (double)vr[j];
      dsr[s] = (float)((double)pr[s] * (dp - dot_sum) * scale);
    } else {
      dsr[s] = 0.f;
    }
  }
  __syncwarp();
  float* dqr = dq + ((size_t)b * T + t) * C + (size_t)h * hd;
  for (int j = lane; j < hd; j += 32) {
    double acc = 0.0;
    for (int s = 0; s <= t; ++s) acc += (double)dsr[s] * (double)k[((size_t)b * T + s) * C + (size_t)h * hd + j];
    dqr[j] = (float)acc;
  }
}

// Per key row: dK[s] = sum_{t>=s} dS[t,s] Q[t], dV[s] = sum_{t>=s} P[t,s] dO[t]; fixed order.
__global__ void attention_f32_bwd_cols_kernel(const float* __restrict__ q, const float* __restrict__ probs,
                                              const float* __restrict__ ds, const float* __restrict__ dout,
                                              float* __restrict__ dk, float* __restrict__ dv, int B, int T, int C, int H) {
  const int hd = C / H;
  const int lane = threadIdx.x & 31;
  const long long w = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)B * H * T) return;
  const int s = (int)(w % T);
  const int h = (int)((w / T) % H);
  const int b = (int)(w / ((long long)T * H));
  const size_t base = ((size_t)b * H + h) * T;
  for (int j = lane; j < hd; j += 32) {
    double ak = 0.0, av = 0.0;
    for (int t = s; t < T; ++t) {
      const size_t pi = (base + t) * (size_t)T + s;
      const size_t xi = ((size_t)b * T + t) * C + (size_t)h * hd + j;
      ak += (double)ds[pi] * (double)q[xi];
      av += (double)probs[pi] * (double)dout[xi];
    }
    const size_t oi = ((size_t)b * T + s) * C + (size_t)h * hd + j;
    dk[oi] = (float)ak;
    dv[oi] = (float)av;
  }
}

int check_attention_dims(int B, int T, int C, int H, const char* who) {
  HL_REQUIRE(H > 0, std::string(who) + ": causal_self_attention requires n_heads > 0");
  HL_REQUIRE(B > 0 && T > 0 && C > 0, std::string(who) + ": batch, time and channels must be positive");
  HL_REQUIRE(C % H == 0, std::string(who) + ": channels " + std::to_string(C) + " must be divisible by n_heads " +
                             std::to_string(H));
  return HL_OK;
}

}  // namespace
}  // namespace hl

using namespace hl;

extern "C" {

int hl_matmul_f32_strided(hl_ctx* ctx, const float* a, const hl_matrix_layout* la, const float* b,
                          const hl_matrix_layout* lb, float* out, const hl_matrix_layout* lo, int accumulate) {
  HL_REQUIRE(ctx && a && la && b && lb && out && lo, "hl_matmul_f32_strided: null argument");
  HL_REQUIRE(la->rows > 0 && la->cols > 0 && lb->cols > 0, "hl_matmul_f32_strided: empty operand");
  HL_REQUIRE(la->cols == lb->rows, "hl_matmul_f32_strided: inner dimensions differ (" + std::to_string(la->cols) +
                                       " vs " + std::to_string(lb->rows) + ")");
  HL_REQUIRE(lo->rows == la->rows && lo->cols == lb->cols, "hl_matmul_f32_strided: output shape mismatch");
  dim3 grid((unsigned)ceil_div_ll(lo->cols, MT), (unsigned)ceil_div_ll(lo->rows, MT)), block(MT, MT);
  HL_REQUIRE(grid.y <= 65535, "hl_matmul_f32_strided: too many rows for one launch");
  matmul_f32_strided_kernel<<<grid, block, 0, ctx->stream>>>(a, *la, b, *lb, out, *lo, accumulate);
  HL_LAUNCH_CHECK("matmul_f32_strided_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_causal_attention_f32_forward(hl_ctx* ctx, const float* q, const float* k, const float* v, float* out,
                                    float* probs, int batch, int time, int channels, int n_heads) {
  HL_REQUIRE(ctx && q && k && v && out && probs, "hl_causal_attention_f32_forward: null argument");
  int rc = check_attention_dims(batch, time, channels, n_heads, "hl_causal_attention_f32_forward");
  if (rc != HL_OK) return rc;
  const long long warps = (long long)batch * n_heads * time;
  attention_f32_fwd_kernel<<<(unsigned)ceil_div_ll(warps, 4), 128, 0, ctx->stream>>>(q, k, v, out, probs, batch, time,
                                                                                    channels, n_heads);
  HL_LAUNCH_CHECK("attention_f32_fwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_causal_attention_f32_backward(hl_ctx* ctx, const float* q, const float* k, const float* v, const float* probs,
                                     const float* grad_out, float* dq, float* dk, float* dv, int batch, int time,
                                     int channels, int n_heads) {
  HL_REQUIRE(ctx && q && k && v && probs && grad_out && dq && dk && dv, "hl_causal_attention_f32_backward: null argument");
  int rc = check_attention_dims(batch, time, channels, n_heads, "hl_causal_attention_f32_backward");
  if (rc != HL_OK) return rc;
  const size_t ds_bytes = sizeof(float) * (size_t)batch * n_heads * time * time;
  rc = ensure_workspace(ctx, ds_bytes);
  if (rc != HL_OK) return rc;
  float* ds = reinterpret_cast<float*>(ctx->workspace);
  const long long warps = (long long)batch * n_heads * time;
  attention_f32_bwd_rows_kernel<<<(unsigned)ceil_div_ll(warps, 4), 128, 0, ctx->stream>>>(k, v, probs, grad_out, ds, dq,
                                                                                         batch, time, channels, n_heads);
  HL_LAUNCH_CHECK("attention_f32_bwd_rows_kernel");
  attention_f32_bwd_cols_kernel<<<(unsigned)ceil_div_ll(warps, 4), 128, 0, ctx->stream>>>(q, probs, ds, grad_out, dk, dv,
                                                                                         batch, time, channels, n_heads);
  HL_LAUNCH_CHECK("attention_f32_bwd_cols_kernel");
  count_launch(ctx, 2);
  return HL_OK;
}

}  // extern "C"
