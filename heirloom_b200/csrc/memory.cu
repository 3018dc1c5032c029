// Product-key memory layer: side scores with the reference's exact f32 dot order, per-token
// top-k selection (ties to the lower index), differentiable re-scoring of the chosen slots,
// weighted value gather and its gradients, row-set AdamW.  One warp per token replaces the
// reference's one-thread-per-token serial selection (heirloom-kernels/src/ptx/kernels.ptx:1780-2262)
// and its one-thread-per-element gathers (:2317-3259); the O(selected^2) duplicate scan of the
// sparse AdamW kernels (:537-811) becomes a row flag pass.
#include "kernels.h"

namespace hl {
namespace {

constexpr float kNegInf = -INFINITY;

// ---- generic per-row top-k (src/tensor.rs:641-702): descending score, ties to the lower index ----
// One warp per row; k rounds of warp arg-max over the lane's strided elements, chosen entries are
// remembered in a per-lane bit set (cols <= 32*64).
__global__ void topk_rows_kernel(const float* __restrict__ scores, int64_t* __restrict__ out, int rows, int cols, int k) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* s = scores + (size_t)row * cols;
  unsigned long long taken = 0ull;  // bit i: element lane + 32*i already chosen
  for (int r = 0; r < k; ++r) {
    float best = kNegInf;
    int best_idx = 0x7fffffff;
    for (int i = 0, c = lane; c < cols; ++i, c += 32) {
      if ((taken >> i) & 1ull) continue;
      const float v = s[c];
      if (best_idx == 0x7fffffff || v > best) { best = v; best_idx = c; }  // strictly greater keeps the lower index
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
      if (oi != 0x7fffffff && (best_idx == 0x7fffffff || ov > best || (ov == best && oi < best_idx))) { best = ov; best_idx = oi; }
    }
    if (best_idx != 0x7fffffff && (best_idx & 31) == lane) taken |= 1ull << (best_idx >> 5);
    if (lane == 0) out[(size_t)row * k + r] = best_idx;
  }
}

// ---- side scores: out[t, s] = sum_j q[t, q_off + j] * keys[s, j], acc = acc + (q*k) in f32 with separately
// rounded multiply and add, j ascending (src/memory_transformer.rs:2029-2034) -------------------------
constexpr int SS_T = 16;  // tokens per block
constexpr int SS_K = 64;  // keys per block
__global__ void __launch_bounds__(256)
side_scores_kernel(const float* __restrict__ query, long long ld_q, int q_off, const float* __restrict__ keys,
                   float* __restrict__ out, int tokens, int side, int half_dim) {
  extern __shared__ float ss_smem[];  // q tile [SS_T][half_dim], key tile transposed [half_dim][SS_K + 1]
  float* sq = ss_smem;
  float* sk = ss_smem + (size_t)SS_T * half_dim;
  const int t0 = blockIdx.y * SS_T, k0 = blockIdx.x * SS_K;
  for (int i = threadIdx.x; i < SS_T * half_dim; i += blockDim.x) {
    const int t = i / half_dim, j = i % half_dim;
    sq[i] = (t0 + t < tokens) ? query[(size_t)(t0 + t) * ld_q + q_off + j] : 0.f;
  }
  for (int i = threadIdx.x; i < SS_K * half_dim; i += blockDim.x) {
    const int kk = i / half_dim, j = i % half_dim;
    sk[(size_t)j * (SS_K + 1) + kk] = (k0 + kk < side) ? keys[(size_t)(k0 + kk) * half_dim + j] : 0.f;
  }
  __syncthreads();
  const int kk = threadIdx.x % SS_K;        // this thread's key
  const int tg = threadIdx.x / SS_K;        // 4 token groups of 4 tokens
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < half_dim; ++j) {
    const float kv = sk[(size_t)j * (SS_K + 1) + kk];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = __fadd_rn(acc[u], __fmul_rn(sq[(size_t)(tg * 4 + u) * half_dim + j], kv));
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int t = t0 + tg * 4 + u;
    if (t < tokens && k0 + kk < side) out[(size_t)t * side + k0 + kk] = acc[u];
  }
}

// ---- product-key candidates from side scores (src/memory_transformer.rs:847-924; CUDA twin
// kernels.ptx:2121-2262): top-`beam` per side (desc score, asc index), beam^2 f32 sums, top-k by
// (desc sum, asc slot).  One warp per token; side <= 2048, beam <= 32, top_k <= beam*beam. ---------
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
  }
}

__global__ void __launch_bounds__(128)
product_key_topk_kernel(const float* __restrict__ left, const float* __restrict__ right, int64_t* __restrict__ out,
                        int tokens, int side, int top_k, int beam, int* __restrict__ status) {
  __shared__ float s_score[4][2][32];
  __shared__ int s_index[4][2][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int token = blockIdx.x * 4 + w;
  if (token >= tokens) return;
  // per side: `beam` rounds of warp arg-max over the lane's strided elements
  for (int sd = 0; sd < 2; ++sd) {
    const float* s = (sd == 0 ? left : right) + (size_t)token * side;
    unsigned long long taken = 0ull;
    for (int r = 0; r < beam; ++r) {
      float best = kNegInf;
      int best_idx = 0x7fffffff;
      for (int i = 0, c = lane; c < side; ++i, c += 32) {
        if ((taken >> i) & 1ull) continue;
        const float v = s[c];
        if (best_idx == 0x7fffffff || v > best) { best = v; best_idx = c; }
      }
      warp_argmax(best, best_idx);
      if (best_idx != 0x7fffffff && (best_idx & 31) == lane) taken |= 1ull << (best_idx >> 5);
      if (lane == 0) { s_score[w][sd][r] = best; s_index[w][sd][r] = best_idx; }
    }
  }
  __syncwarp();
  // candidates: lane owns left entry `lane` (if < beam) against every right entry
  const bool has = lane < beam;
  const float ls = has ? s_score[w][0][lane] : 0.f;
  const int li = has ? s_index[w][0][lane] : 0;
  unsigned int used = 0u;  // bit r: candidate (lane, r) already chosen
  for (int r = 0; r < top_k; ++r) {
    float best = kNegInf;
    int best_slot = 0x7fffffff;
    if (has) {
      for (int j = 0; j < beam; ++j) {
        if ((used >> j) & 1u) continue;
        const float v = __fadd_rn(ls, s_score[w][1][j]);
        const int slot = li * side + s_index[w][1][j];
        if (best_slot == 0x7fffffff || v > best || (v == best && slot < best_slot)) { best = v; best_slot = slot; }
      }
    }
    float bv = best;
    int bs = best_slot;
    warp_argmax(bv, bs);
    if (bs == 0x7fffffff) {
      if (lane == 0) { atomicExch(status + ST_BAD_ARGUMENT, 1); out[(size_t)token * top_k + r] = 0; }
      continue;
    }
    if (has && bs / side == li) {  // the winner is one of this lane's candidates: retire it
      const int rj = bs % side;
      for (int j = 0; j < beam; ++j)
        if (s_index[w][1][j] == rj) used |= 1u << j;
    }
    if (lane == 0) out[(size_t)token * top_k + r] = bs;
  }
}

__global__ void split_rows_kernel(const int64_t* __restrict__ rows, int64_t* __restrict__ left, int64_t* __restrict__ right,
                                  long long n, int side) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long r = rows[i];
  left[i] = r / side;
  right[i] = r % side;
}

// ---- selected scores: score[t,k] = q_L . K_L[idx/side] + q_R . K_R[idx%side]  (src/tensor.rs:3593-3769).
// `exact` mode (side == 0): score = q . K[idx] over key_dim (src/tensor.rs:3465-3548). One warp per token. ---
__global__ void selected_scores_fwd_kernel(const int64_t* __restrict__ idx, const float* __restrict__ query, long long ld_q,
                                           const float* __restrict__ left, const float* __restrict__ right,
                                           float* __restrict__ scores, int tokens, int top_k, int side, int key_dim,
                                           int slots, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const int half = side > 0 ? key_dim / 2 : key_dim;
  const float* q = query + (size_t)token * ld_q;
  for (int k = 0; k < top_k; ++k) {
    const long long slot = idx[(size_t)token * top_k + k];
    if (slot < 0 || slot >= slots) {
      if (lane == 0) { atomicExch(status + ST_BAD_INDEX, 1); scores[(size_t)token * top_k + k] = 0.f; }
      continue;
    }
    double acc = 0.0;
    if (side > 0) {
      const float* kl = left + (size_t)(slot / side) * half;
      const float* kr = right + (size_t)(slot % side) * half;
      for (int j = lane; j < half; j += 32) acc += (double)q[j] * (double)kl[j] + (double)q[half + j] * (double)kr[j];
    } else {
      const float* kr = left + (size_t)slot * key_dim;
      for (int j = lane; j < key_dim; j += 32) acc += (double)q[j] * (double)kr[j];
    }
    acc = warp_sum(acc);
    if (lane == 0) scores[(size_t)token * top_k + k] = (float)acc;
  }
}

// dq[t,:] = sum_k g[t,k] * [K_L[li]; K_R[ri]]; dK_L[li,:] += g[t,k] q_L[t]; dK_R[ri,:] += g[t,k] q_R[t]
// (src/tensor/autograd.rs:2386-2494).  Key gradients use f32 atomics like the reference.
__global__ void selected_scores_bwd_kernel(const int64_t* __restrict__ idx, const float* __restrict__ query, long long ld_q,
                                           const float* __restrict__ left, const float* __restrict__ right,
                                           const float* __restrict__ grad_scores, float* __restrict__ dq, long long ld_dq,
                                           float* __restrict__ dleft, float* __restrict__ dright, int tokens, int top_k,
                                           int side, int key_dim, int slots) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const int half = side > 0 ? key_dim / 2 : key_dim;
  const float* q = query + (size_t)token * ld_q;
  for (int j = lane; j < key_dim; j += 32) {
    double acc = 0.0;
    for (int k = 0; k < top_k; ++k) {
      const long long slot = idx[(size_t)token * top_k + k];
      if (slot < 0 || slot >= slots) continue;
      const double g = (double)grad_scores[(size_t)token * top_k + k];
      float kv;
      if (side > 0) kv = j < half ? left[(size_t)(slot / side) * half + j] : right[(size_t)(slot % side) * half + (j - half)];
      else kv = left[(size_t)slot * key_dim + j];
      acc += g * (double)kv;
    }
    if (dq) dq[(size_t)token * ld_dq + j] = (float)acc;
  }
  for (int k = 0; k < top_k; ++k) {
    const long long slot = idx[(size_t)token * top_k + k];
    if (slot < 0 || slot >= slots) continue;
    const float g = grad_scores[(size_t)token * top_k + k];
    if (side > 0) {
      float* dl = dleft + (size_t)(slot / side) * half;
      float* dr = dright + (size_t)(slot % side) * half;
      for (int j = lane; j < half; j += 32) {
        if (dleft) atomicAdd(dl + j, g * q[j]);
        if (dright) atomicAdd(dr + j, g * q[half + j]);
      }
    } else if (dleft) {
      float* dk = dleft + (size_t)slot * key_dim;
      for (int j = lane; j < key_dim; j += 32) atomicAdd(dk + j, g * q[j]);
    }
  }
}

// ---- row softmax over a few columns (top-k weights), src/tensor.rs:4521-4602 / autograd.rs:2512-2543 ----
__global__ void softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* xr = x + (size_t)row * cols;
  double mx = -INFINITY;
  for (int c = lane; c < cols; c += 32) mx = max(mx, (double)xr[c]);
  mx = warp_max(mx);
  double s = 0.0;
  for (int c = lane; c < cols; c += 32) s += exp((double)xr[c] - mx);
  s = warp_sum(s);
  for (int c = lane; c < cols; c += 32) y[(size_t)row * cols + c] = (float)(exp((double)xr[c] - mx) / s);
}

__global__ void softmax_rows_bwd_kernel(const float* __restrict__ y, const float* __restrict__ gy, float* __restrict__ gx,
                                        int rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  double dot = 0.0;
  for (int c = lane; c < cols; c += 32) dot += (double)y[(size_t)row * cols + c] * (double)gy[(size_t)row * cols + c];
  dot = warp_sum(dot);
  for (int c = lane; c < cols; c += 32) {
    const size_t i = (size_t)row * cols + c;
    gx[i] = (float)((double)y[i] * ((double)gy[i] - dot));
  }
}

// ---- weighted value: out[t,:] = sum_k w[t,k] V[idx[t,k],:] (* gate[t,:] when given)  (src/tensor.rs:3771-3900).
// One warp per token, 128-bit row gathers. ------------------------------------------------------------
__global__ void weighted_value_fwd_kernel(const int64_t* __restrict__ idx, const float* __restrict__ weights,
                                          const float* __restrict__ values, float* __restrict__ out, int tokens, int top_k,
                                          int rows, int dim, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= tokens) return;
  for (int c = lane * 4; c < dim; c += 128) {
    double a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    for (int k = 0; k < top_k; ++k) {
      const long long r = idx[(size_t)token * top_k + k];
      if (r < 0 || r >= rows) { if (lane == 0 && c == 0) atomicExch(status + ST_BAD_INDEX, 1); continue; }
      const double w = (double)weights[(size_t)token * top_k + k];
      const float4 v = __ldg(reinterpret_cast<const float4*>(values + (size_t)r * dim + c));
      a0 += w * v.x; a1 += w * v.y; a2 += w * v.z; a3 += w * v.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)token * dim + c) = make_float4((float)a0, (float)a1, (float)a2, (float)a3);
  }
}

// dw[t,k] = dout[t] . V[idx[t,k]];  dV[idx[t,k],:] += w[t,k] dout[t,:] (f32 atomics, repeats accumulate)
// (src/tensor/autograd.rs:2263-2323).
__global__ void weighted_value_bwd_kernel(const int64_t* __restrict__ idx, const float* __restrict__ weights,
                                          const float* __restrict__ values, const float* __restrict__ grad_out,
                                          float* __restrict__ dweights, float* __restrict__ dvalues, int tokens, int top_k,
                                          int rows, int dim) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const float* go = grad_out + (size_t)token * dim;
  for (int k = 0; k < top_k; ++k) {
    const long long r = idx[(size_t)token * top_k + k];
    if (r < 0 || r >= rows) continue;
    const float w = weights[(size_t)token * top_k + k];
    double dot = 0.0;
    for (int c = lane * 4; c < dim; c += 128) {
      const float4 g = *reinterpret_cast<const float4*>(go + c);
      if (dweights) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(values + (size_t)r * dim + c));
        dot += (double)g.x * v.x + (double)g.y * v.y + (double)g.z * v.z + (double)g.w * v.w;
      }
      if (dvalues) atomicAdd(reinterpret_cast<float4*>(dvalues + (size_t)r * dim + c), make_float4(w * g.x, w * g.y, w * g.z, w * g.w));
    }
    if (dweights) {
      dot = warp_sum(dot);
      if (lane == 0) dweights[(size_t)token * top_k + k] = (float)dot;
    }
  }
}

// ---- row-set AdamW (src/nn.rs:2256-2323, :2899-2939; kernels.ptx:537-811) -----------------------------------
__global__ void mark_rows_kernel(const int64_t* __restrict__ selected, long long n, unsigned char* __restrict__ flags,
                                 const unsigned char* __restrict__ row_mask, int rows, int* __restrict__ status) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long r = selected[i];
  if (r < 0 || r >= rows) { atomicExch(status + ST_BAD_INDEX, 1); return; }
  if (row_mask == nullptr || row_mask[r]) flags[r] = 1;
}

__device__ __forceinline__ void adamw_one(float& p, float g, float& m, float& v, const hl_adamw_params& hp) {
  const float gd = __fadd_rn(__fmul_rn(g, hp.clip_scale), __fmul_rn(p, hp.weight_decay));
  m = __fadd_rn(__fmul_rn(hp.beta1, m), __fmul_rn(__fsub_rn(1.0f, hp.beta1), gd));
  v = __fadd_rn(__fmul_rn(hp.beta2, v), __fmul_rn(__fsub_rn(1.0f, hp.beta2), __fmul_rn(gd, gd)));
  const float upd = __fdiv_rn(__fdiv_rn(m, hp.bias_correction1), __fadd_rn(__fsqrt_rn(__fdiv_rn(v, hp.bias_correction2)), hp.eps));
  p = __fsub_rn(p, __fmul_rn(hp.lr, upd));
}

// One warp per flagged row; clears the flag and (optionally) the gradient row it consumed.
__global__ void sparse_adamw_rows_kernel(float* __restrict__ param, float* __restrict__ grad, float* __restrict__ m,
                                         float* __restrict__ v, unsigned char* __restrict__ flags, int rows, int row_dim,
                                         const hl_adamw_params hp, int zero_grad_rows) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows || !flags[row]) return;
  const size_t base = (size_t)row * row_dim;
  for (int c = lane; c < row_dim; c += 32) {
    float p = param[base + c], mm = m[base + c], vv = v[base + c];
    adamw_one(p, grad[base + c], mm, vv, hp);
    param[base + c] = p; m[base + c] = mm; v[base + c] = vv;
    if (zero_grad_rows) grad[base + c] = 0.f;
  }
  __syncwarp();
  if (lane == 0) flags[row] = 0;
}

int check_memory_dims(int tokens, int top_k, int dim, const char* who) {
  HL_REQUIRE(tokens > 0 && top_k > 0 && dim > 0, std::string(who) + ": requires non-zero tokens/top_k/dim");
  return HL_OK;
}

}  // namespace
}  // namespace hl

using namespace hl;

extern "C" {

int hl_topk_rows_f32(hl_ctx* ctx, const float* scores, int64_t* out, int rows, int cols, int k) {
  HL_REQUIRE(ctx && scores && out, "hl_topk_rows_f32: null argument");
  HL_REQUIRE(rows > 0 && cols > 0, "hl_topk_rows_f32: requires non-zero rows/cols");
  HL_REQUIRE(k > 0 && k <= cols, "hl_topk_rows_f32: k must be in [1, cols]");
  HL_REQUIRE(cols <= 2048, "hl_topk_rows_f32: at most 2048 columns");
  topk_rows_kernel<<<ceil_div(rows, 4), 128, 0, ctx->stream>>>(scores, out, rows, cols, k);
  HL_LAUNCH_CHECK("topk_rows_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_product_key_side_scores_f32(hl_ctx* ctx, const float* query, long long ld_query, const float* left_keys,
                                   const float* right_keys, float* left_scores, float* right_scores, int tokens, int side,
                                   int key_dim) {
  HL_REQUIRE(ctx && query && left_keys && right_keys && left_scores && right_scores, "hl_product_key_side_scores_f32: null argument");
  HL_REQUIRE(tokens > 0 && side > 0 && key_dim > 0, "hl_product_key_side_scores_f32: requires non-zero sizes");
  HL_REQUIRE(key_dim % 2 == 0, "product-key memory lookup requires even memory_key_dim, got " + std::to_string(key_dim));
  HL_REQUIRE(ld_query >= key_dim, "hl_product_key_side_scores_f32: query row stride smaller than key_dim");
  const int half = key_dim / 2;
  const size_t smem = sizeof(float) * ((size_t)SS_T * half + (size_t)half * (SS_K + 1));
  HL_REQUIRE(smem <= 200 * 1024, "hl_product_key_side_scores_f32: key_dim too large for one shared-memory tile");
  HL_CUDA(cudaFuncSetAttribute(side_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(ceil_div(side, SS_K), ceil_div(tokens, SS_T));
  side_scores_kernel<<<grid, 256, smem, ctx->stream>>>(query, ld_query, 0, left_keys, left_scores, tokens, side, half);
  HL_LAUNCH_CHECK("side_scores_kernel");
  side_scores_kernel<<<grid, 256, smem, ctx->stream>>>(query, ld_query, half, right_keys, right_scores, tokens, side, half);
  HL_LAUNCH_CHECK("side_scores_kernel");
  count_launch(ctx, 2);
  return HL_OK;
}

int hl_product_key_topk_from_side_scores(hl_ctx* ctx, const float* left_scores, const float* right_scores, int64_t* out,
                                         int tokens, int side, int top_k, int beam) {
  HL_REQUIRE(ctx && left_scores && right_scores && out, "hl_product_key_topk_from_side_scores: null argument");
  HL_REQUIRE(tokens > 0 && side > 0, "hl_product_key_topk_from_side_scores: requires non-zero tokens/side");
  HL_REQUIRE(side <= 2048, "hl_product_key_topk_from_side_scores: side must be at most 2048");
  HL_REQUIRE(beam > 0 && beam <= 32 && beam <= side, "hl_product_key_topk_from_side_scores: beam must be in [1, min(32, side)]");
  HL_REQUIRE(top_k > 0 && top_k <= beam * beam, "hl_product_key_topk_from_side_scores: top_k must be in [1, beam^2]");
  product_key_topk_kernel<<<ceil_div(tokens, 4), 128, 0, ctx->stream>>>(left_scores, right_scores, out, tokens, side, top_k,
                                                                        beam, ctx->status_dev);
  HL_LAUNCH_CHECK("product_key_topk_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_product_key_split_rows(hl_ctx* ctx, const int64_t* rows, int64_t* left, int64_t* right, long long n, int side) {
  HL_REQUIRE(ctx && rows && left && right, "hl_product_key_split_rows: null argument");
  HL_REQUIRE(n > 0 && side > 0, "hl_product_key_split_rows: requires non-zero rows/side");
  split_rows_kernel<<<(unsigned)ceil_div_ll(n, 256), 256, 0, ctx->stream>>>(rows, left, right, n, side);
  HL_LAUNCH_CHECK("split_rows_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_memory_selected_scores_forward(hl_ctx* ctx, const int64_t* indices, const float* query, long long ld_query,
                                      const float* left_or_keys, const float* right_keys, float* scores, int tokens,
                                      int top_k, int side, int key_dim, int slots) {
  HL_REQUIRE(ctx && indices && query && left_or_keys && scores, "hl_memory_selected_scores_forward: null argument");
  int rc = check_memory_dims(tokens, top_k, key_dim, "hl_memory_selected_scores_forward");
  if (rc != HL_OK) return rc;
  HL_REQUIRE(side == 0 || (right_keys && key_dim % 2 == 0 && (long long)side * side == slots),
             "hl_memory_selected_scores_forward: product-key mode needs both half tables, even key_dim and square slots");
  selected_scores_fwd_kernel<<<ceil_div(tokens, 4), 128, 0, ctx->stream>>>(indices, query, ld_query, left_or_keys, right_keys,
                                                                           scores, tokens, top_k, side, key_dim, slots,
                                                                           ctx->status_dev);
  HL_LAUNCH_CHECK("selected_scores_fwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_memory_selected_scores_backward(hl_ctx* ctx, const int64_t* indices, const float* query, long long ld_query,
                                       const float* left_or_keys, const float* right_keys, const float* grad_scores,
                                       float* grad_query, long long ld_grad_query, float* grad_left_or_keys,
                                       float* grad_right_keys, int tokens, int top_k, int side, int key_dim, int slots) {
  HL_REQUIRE(ctx && indices && query && left_or_keys && grad_scores, "hl_memory_selected_scores_backward: null argument");
  int rc = check_memory_dims(tokens, top_k, key_dim, "hl_memory_selected_scores_backward");
  if (rc != HL_OK) return rc;
  HL_REQUIRE(side == 0 || (right_keys && key_dim % 2 == 0), "hl_memory_selected_scores_backward: product-key mode needs both half tables");
  selected_scores_bwd_kernel<<<ceil_div(tokens, 4), 128, 0, ctx->stream>>>(
      indices, query, ld_query, left_or_keys, right_keys, grad_scores, grad_query, ld_grad_query, grad_left_or_keys,
      grad_right_keys, tokens, top_k, side, key_dim, slots);
  HL_LAUNCH_CHECK("selected_scores_bwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_softmax_rows_f32(hl_ctx* ctx, const float* x, float* y, int rows, int cols) {
  HL_REQUIRE(ctx && x && y, "hl_softmax_rows_f32: null argument");
  HL_REQUIRE(rows > 0 && cols > 0, "hl_softmax_rows_f32: requires non-zero rows/cols");
  softmax_rows_kernel<<<ceil_div(rows, 4), 128, 0, ctx->stream>>>(x, y, rows, cols);
  HL_LAUNCH_CHECK("softmax_rows_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_softmax_rows_backward_f32(hl_ctx* ctx, const float* y, const float* grad_y, float* grad_x, int rows, int cols) {
  HL_REQUIRE(ctx && y && grad_y && grad_x, "hl_softmax_rows_backward_f32: null argument");
  HL_REQUIRE(rows > 0 && cols > 0, "hl_softmax_rows_backward_f32: requires non-zero rows/cols");
  softmax_rows_bwd_kernel<<<ceil_div(rows, 4), 128, 0, ctx->stream>>>(y, grad_y, grad_x, rows, cols);
  HL_LAUNCH_CHECK("softmax_rows_bwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_memory_weighted_value_forward(hl_ctx* ctx, const int64_t* indices, const float* weights, const float* values,
                                     float* out, int tokens, int top_k, int rows, int dim) {
  HL_REQUIRE(ctx && indices && weights && values && out, "hl_memory_weighted_value_forward: null argument");
  int rc = check_memory_dims(tokens, top_k, dim, "hl_memory_weighted_value_forward");
  if (rc != HL_OK) return rc;
  HL_REQUIRE(rows > 0 && dim % 4 == 0, "hl_memory_weighted_value_forward: non-zero rows/row_dim, row_dim a multiple of 4");
  weighted_value_fwd_kernel<<<ceil_div(tokens, 4), 128, 0, ctx->stream>>>(indices, weights, values, out, tokens, top_k, rows,
                                                                          dim, ctx->status_dev);
  HL_LAUNCH_CHECK("weighted_value_fwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_memory_weighted_value_backward(hl_ctx* ctx, const int64_t* indices, const float* weights, const float* values,
                                      const float* grad_out, float* grad_weights, float* grad_values, int tokens,
                                      int top_k, int rows, int dim) {
  HL_REQUIRE(ctx && indices && weights && values && grad_out, "hl_memory_weighted_value_backward: null argument");
  int rc = check_memory_dims(tokens, top_k, dim, "hl_memory_weighted_value_backward");
  if (rc != HL_OK) return rc;
  HL_REQUIRE(rows > 0 && dim % 4 == 0, "hl_memory_weighted_value_backward: non-zero rows/row_dim, row_dim a multiple of 4");
  weighted_value_bwd_kernel<<<ceil_div(tokens, 4), 128, 0, ctx->stream>>>(indices, weights, values, grad_out, grad_weights,
                                                                          grad_values, tokens, top_k, rows, dim);
  HL_LAUNCH_CHECK("weighted_value_bwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_sparse_adamw_rows_f32(hl_ctx* ctx, float* param, float* grad, float* m, float* v, const int64_t* selected_rows,
                             long long n_selected, const unsigned char* row_mask, unsigned char* row_flags, int rows,
                             int row_dim, const hl_adamw_params* hp, int zero_grad_rows) {
  HL_REQUIRE(ctx && param && grad && m && v && selected_rows && row_flags && hp, "hl_sparse_adamw_rows_f32: null argument");
  HL_REQUIRE(rows > 0 && row_dim > 0, "hl_sparse_adamw_rows_f32: requires non-zero rows/row_dim");
  HL_REQUIRE(hp->bias_correction1 > 0.f && hp->bias_correction2 > 0.f, "hl_sparse_adamw_rows_f32: bias corrections must be positive");
  if (n_selected <= 0) return HL_OK;
  mark_rows_kernel<<<(unsigned)ceil_div_ll(n_selected, 256), 256, 0, ctx->stream>>>(selected_rows, n_selected, row_flags,
                                                                                  row_mask, rows, ctx->status_dev);
  HL_LAUNCH_CHECK("mark_rows_kernel");
  sparse_adamw_rows_kernel<<<ceil_div(rows, 8), 256, 0, ctx->stream>>>(param, grad, m, v, row_flags, rows, row_dim, *hp,
                                                                       zero_grad_rows);
  HL_LAUNCH_CHECK("sparse_adamw_rows_kernel");
  count_launch(ctx, 2);
  return HL_OK;
}

}  // extern "C"
