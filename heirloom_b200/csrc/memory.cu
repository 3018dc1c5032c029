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
// Block tile 64 tokens x 128 keys, thread tile 8 tokens x 4 keys; the contraction walks in slices of 64 that are
// staged in shared memory (queries as [j][token], keys as [j][key]), so a step of the inner loop is three 16-byte
// shared-memory loads for 32 multiplies and 32 adds.  Every accumulator still sees j = 0, 1, 2, ... in order.
constexpr int SS_T = 64;   // tokens per block
constexpr int SS_K = 128;  // keys per block
constexpr int SS_J = 64;   // contraction slice
__global__ void __launch_bounds__(256)
side_scores_kernel(const float* __restrict__ query, long long ld_q, int q_off, const float* __restrict__ keys,
                   float* __restrict__ out, int tokens, int side, int half_dim) {
  __shared__ __align__(16) float sq[SS_J][SS_T];
  __shared__ __align__(16) float sk[SS_J][SS_K];
  const int t0 = blockIdx.y * SS_T, k0 = blockIdx.x * SS_K;
  const int ty = threadIdx.x >> 5;  // 8 token groups of 8 tokens
  const int tx = threadIdx.x & 31;  // 32 key groups of 4 keys
  float acc[8][4];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  for (int j0 = 0; j0 < half_dim; j0 += SS_J) {
    // stage the slice: consecutive threads read consecutive j of one row (coalesced), and write transposed
    for (int i = threadIdx.x; i < SS_T * SS_J; i += 256) {
      const int t = i / SS_J, j = i % SS_J;
      sq[j][t] = (t0 + t < tokens && j0 + j < half_dim) ? query[(size_t)(t0 + t) * ld_q + q_off + j0 + j] : 0.f;
    }
    for (int i = threadIdx.x; i < SS_K * SS_J; i += 256) {
      const int kk = i / SS_J, j = i % SS_J;
      sk[j][kk] = (k0 + kk < side && j0 + j < half_dim) ? keys[(size_t)(k0 + kk) * half_dim + j0 + j] : 0.f;
    }
    __syncthreads();
    const int jn = min(SS_J, half_dim - j0);
    for (int j = 0; j < jn; ++j) {
      const float4 qa = *reinterpret_cast<const float4*>(&sq[j][ty * 8]);
      const float4 qb = *reinterpret_cast<const float4*>(&sq[j][ty * 8 + 4]);
      const float4 kv = *reinterpret_cast<const float4*>(&sk[j][tx * 4]);
      const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
      const float kk4[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = __fadd_rn(acc[a][b], __fmul_rn(qv[a], kk4[b]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int t = t0 + ty * 8 + a;
    if (t >= tokens) continue;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int kk = k0 + tx * 4 + b;
      if (kk < side) out[(size_t)t * side + kk] = acc[a][b];
    }
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

// Values stay in registers: a lane keeps its strided side scores (up to 64 per side, side <= 2048) and its own
// current best; a round is one warp arg-max over the lanes' bests, after which only the winning lane rescans.
constexpr int PK_MAX_PER_LANE = 64;
template <int PER_LANE>
__device__ __forceinline__ void lane_best(const float (&v)[PER_LANE], unsigned long long taken, int n, int lane,
                                          float* best, int* best_idx) {
  *best = kNegInf;
  *best_idx = 0x7fffffff;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    if (i < n && !((taken >> i) & 1ull) && (*best_idx == 0x7fffffff || v[i] > *best)) {
      *best = v[i];
      *best_idx = i * 32 + lane;  // ascending index within the lane, so the first maximum is the lowest index
    }
  }
}

template <int PER_LANE>
__global__ void __launch_bounds__(128)
product_key_topk_kernel(const float* __restrict__ left, const float* __restrict__ right, int64_t* __restrict__ out,
                        int tokens, int side, int top_k, int beam, int* __restrict__ status) {
  __shared__ float s_score[4][2][32];
  __shared__ int s_index[4][2][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int token = blockIdx.x * 4 + w;
  if (token >= tokens) return;
  const int n_mine = (side - lane + 31) / 32;  // entries lane, lane+32, ... below side
  // per side: `beam` rounds of warp arg-max (desc score, asc index)
  for (int sd = 0; sd < 2; ++sd) {
    const float* s = (sd == 0 ? left : right) + (size_t)token * side;
    float v[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) v[i] = (i < n_mine) ? s[i * 32 + lane] : kNegInf;
    unsigned long long taken = 0ull;
    float mine;
    int mine_idx;
    lane_best<PER_LANE>(v, taken, n_mine, lane, &mine, &mine_idx);
    for (int r = 0; r < beam; ++r) {
      float best = mine;
      int best_idx = mine_idx;
      warp_argmax(best, best_idx);
      if (best_idx != 0x7fffffff && (best_idx & 31) == lane) {
        taken |= 1ull << (best_idx >> 5);
        lane_best<PER_LANE>(v, taken, n_mine, lane, &mine, &mine_idx);
      }
      if (lane == 0) { s_score[w][sd][r] = best; s_index[w][sd][r] = best_idx; }
    }
  }
  __syncwarp();
  // candidates: lane owns left entry `lane` (if < beam) against every right entry; sums and slots in registers
  const bool has = lane < beam;
  const float ls = has ? s_score[w][0][lane] : 0.f;
  const int li = has ? s_index[w][0][lane] : 0;
  float cand[32];
  int cslot[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const bool live = has && j < beam;
    cand[j] = live ? __fadd_rn(ls, s_score[w][1][j]) : kNegInf;
    cslot[j] = live ? li * side + s_index[w][1][j] : 0x7fffffff;
  }
  unsigned int used = 0u;  // bit j: candidate (lane, j) already chosen
  auto rescan = [&](float* best, int* best_slot) {
    *best = kNegInf;
    *best_slot = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (cslot[j] == 0x7fffffff || ((used >> j) & 1u)) continue;
      if (*best_slot == 0x7fffffff || cand[j] > *best || (cand[j] == *best && cslot[j] < *best_slot)) {
        *best = cand[j];
        *best_slot = cslot[j];
      }
    }
  };
  float mine;
  int mine_slot;
  rescan(&mine, &mine_slot);
  for (int r = 0; r < top_k; ++r) {
    float bv = mine;
    int bs = mine_slot;
    warp_argmax(bv, bs);
    if (bs == 0x7fffffff) {
      if (lane == 0) { atomicExch(status + ST_BAD_ARGUMENT, 1); out[(size_t)token * top_k + r] = 0; }
      continue;
    }
    if (has && bs == mine_slot) {  // the winner is this lane's candidate: retire it and rescan
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (cslot[j] == bs) used |= 1u << j;
      rescan(&mine, &mine_slot);
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
  if (side > 0) return;  // the half-key gradients of the product-key form come from product_key_dkeys_kernel
  for (int k = 0; k < top_k; ++k) {
    const long long slot = idx[(size_t)token * top_k + k];
    if (slot < 0 || slot >= slots) continue;
    const float g = grad_scores[(size_t)token * top_k + k];
    if (dleft) {
      float* dk = dleft + (size_t)slot * key_dim;
      for (int j = lane; j < key_dim; j += 32) atomicAdd(dk + j, g * q[j]);
    }
  }
}

// Half-key gradients of the product-key form: dK_L[li,:] += g[t,k] q_L[t,:], dK_R[ri,:] += g[t,k] q_R[t,:] over the
// selected slots.  With only `side` rows per table every row collects about tokens*top_k/side terms, so atomics
// (global or shared) would pile onto a few addresses.  The sum is therefore run as a dense product
// dK = Wᵀ·Q with W[t, row] = sum of the g[t,k] whose slot maps to `row`: a CTA owns a block of tokens, 512 rows
// and 64 columns of one table; per slice of 32 tokens it builds W in shared memory (one warp per token, its
// duplicates added in slot order), multiplies with a 16 x 8 register tile per thread, and clears the entries it
// set.  The CTA's tile goes out as a partial result that fold_key_partials_kernel adds up in block order, so the
// result does not depend on scheduling.
constexpr int DK_COLS = 64;    // columns per CTA
constexpr int DK_ROWS = 512;   // table rows per CTA
constexpr int DK_TOKENS = 32;  // tokens per slice
__global__ void __launch_bounds__(256)
product_key_dkeys_kernel(const int64_t* __restrict__ idx, const float* __restrict__ query, long long ld_q,
                         const float* __restrict__ grad_scores, float* __restrict__ partial, int tokens, int top_k,
                         int side, int half, int slots, int tokens_per_block, int col_blocks) {
  extern __shared__ __align__(16) float dk_smem[];
  float* w_tile = dk_smem;                          // [DK_TOKENS][DK_ROWS]
  float* q_tile = dk_smem + DK_TOKENS * DK_ROWS;    // [DK_TOKENS][DK_COLS]
  const int table = blockIdx.z;                     // 0 left, 1 right
  const int c0 = (blockIdx.y % col_blocks) * DK_COLS;
  const int r0 = (blockIdx.y / col_blocks) * DK_ROWS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tr = threadIdx.x >> 3;  // 32 row groups of 16 rows
  const int tc = threadIdx.x & 7;   // 8 column groups of 8 columns
  float acc[16][8];
#pragma unroll
  for (int a = 0; a < 16; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0.f;
  for (int i = threadIdx.x; i < DK_TOKENS * DK_ROWS; i += 256) w_tile[i] = 0.f;
  const int t_begin = blockIdx.x * tokens_per_block, t_end = min(tokens, t_begin + tokens_per_block);
  for (int t0 = t_begin; t0 < t_end; t0 += DK_TOKENS) {
    __syncthreads();  // the previous slice's product is done (and, first time, the tile is zero)
    // this slice's query columns
    for (int i = threadIdx.x; i < DK_TOKENS * DK_COLS; i += 256) {
      const int t = i / DK_COLS, c = i % DK_COLS;
      q_tile[i] = (t0 + t < t_end && c0 + c < half) ? query[(size_t)(t0 + t) * ld_q + (table ? half : 0) + c0 + c] : 0.f;
    }
    // W rows: warp w builds tokens w, w+8, ...; lane 0 adds the token's gradients in slot order
    for (int t = warp; t < DK_TOKENS; t += 8) {
      if (t0 + t >= t_end) break;
      for (int k0 = 0; k0 < top_k; k0 += 32) {
        long long my_slot = -1;
        float my_g = 0.f;
        if (k0 + lane < top_k) {
          my_slot = idx[(size_t)(t0 + t) * top_k + k0 + lane];
          my_g = grad_scores[(size_t)(t0 + t) * top_k + k0 + lane];
        }
        const int n = min(32, top_k - k0);
        for (int k = 0; k < n; ++k) {
          const long long slot = __shfl_sync(0xffffffffu, my_slot, k);
          const float g = __shfl_sync(0xffffffffu, my_g, k);
          if (slot < 0 || slot >= slots) continue;
          const int row = (table ? (int)(slot % side) : (int)(slot / side)) - r0;
          if (lane == 0 && row >= 0 && row < DK_ROWS) w_tile[t * DK_ROWS + row] += g;
        }
      }
    }
    __syncthreads();
    const int tn = min(DK_TOKENS, t_end - t0);
    for (int t = 0; t < tn; ++t) {
      float wv[16], qv[8];
#pragma unroll
      for (int a = 0; a < 16; a += 4) {
        const float4 x = *reinterpret_cast<const float4*>(&w_tile[t * DK_ROWS + tr * 16 + a]);
        wv[a] = x.x; wv[a + 1] = x.y; wv[a + 2] = x.z; wv[a + 3] = x.w;
      }
#pragma unroll
      for (int b = 0; b < 8; b += 4) {
        const float4 x = *reinterpret_cast<const float4*>(&q_tile[t * DK_COLS + tc * 8 + b]);
        qv[b] = x.x; qv[b + 1] = x.y; qv[b + 2] = x.z; qv[b + 3] = x.w;
      }
#pragma unroll
      for (int a = 0; a < 16; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(wv[a], qv[b], acc[a][b]);
    }
    __syncthreads();
    // clear what this slice set
    for (int t = warp; t < DK_TOKENS; t += 8) {
      if (t0 + t >= t_end) break;
      for (int k = lane; k < top_k; k += 32) {
        const long long slot = idx[(size_t)(t0 + t) * top_k + k];
        if (slot < 0 || slot >= slots) continue;
        const int row = (table ? (int)(slot % side) : (int)(slot / side)) - r0;
        if (row >= 0 && row < DK_ROWS) w_tile[t * DK_ROWS + row] = 0.f;
      }
    }
  }
  // partial[block][table][side][half]
  float* dst = partial + ((size_t)blockIdx.x * 2 + table) * side * half;
#pragma unroll
  for (int a = 0; a < 16; ++a) {
    const int row = r0 + tr * 16 + a;
    if (row >= side) continue;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int c = c0 + tc * 8 + b;
      if (c < half) dst[(size_t)row * half + c] = acc[a][b];
    }
  }
}

__global__ void fold_key_partials_kernel(const float* __restrict__ partial, float* __restrict__ dleft,
                                         float* __restrict__ dright, int blocks, int side, int half) {
  const size_t per_table = (size_t)side * half;
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= 2 * per_table) return;
  const int table = i >= per_table;
  const size_t e = i - table * per_table;
  float* dst = table ? dright : dleft;
  if (!dst) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[((size_t)b * 2 + table) * per_table + e];
  dst[e] += s;  // the tables are shared by every memory block of the model: gradients accumulate
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

// Sum of squares of the flagged gradient rows (a set: a row counts once however often it was selected); one
// warp per flagged row, f64 partial per warp, flags cleared on the way out.
__global__ void flagged_rows_sum_squares_kernel(const float* __restrict__ grad, unsigned char* __restrict__ flags, int rows,
                                                int row_dim, double* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows || !flags[row]) return;
  const float* g = grad + (size_t)row * row_dim;
  double s = 0.0;
  for (int c = lane; c < row_dim; c += 32) s += (double)g[c] * (double)g[c];
  s = warp_sum(s);
  __syncwarp();
  if (lane == 0) {
    atomicAdd(out, s);
    flags[row] = 0;
  }
}

// Ascending indices of the non-zero bytes of a mask, and their count.  One CTA: every thread counts a contiguous
// span, an exclusive scan over the spans gives its write position.
__global__ void __launch_bounds__(1024)
mask_to_indices_kernel(const unsigned char* __restrict__ mask, int rows, int64_t* __restrict__ out, int* __restrict__ count) {
  __shared__ int span_start[1025];
  const int per = (rows + 1023) / 1024;
  const int lo = min(rows, (int)threadIdx.x * per), hi = min(rows, lo + per);
  int mine = 0;
  for (int r = lo; r < hi; ++r) mine += mask[r] != 0;
  span_start[threadIdx.x + 1] = mine;
  if (threadIdx.x == 0) span_start[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0)
    for (int i = 1; i <= 1024; ++i) span_start[i] += span_start[i - 1];
  __syncthreads();
  int at = span_start[threadIdx.x];
  for (int r = lo; r < hi; ++r)
    if (mask[r]) out[at++] = r;
  if (threadIdx.x == 0) *count = span_start[1024];
}

// dst[i,:] = src[idx[i],:] (gather) or dst[idx[i],:] = src[i,:] (scatter); one warp per row, 16-byte accesses.
__global__ void move_rows_kernel(const float* __restrict__ src, const int64_t* __restrict__ idx, const int* __restrict__ count_dev,
                                 int n_max, int dim, float* __restrict__ dst, int scatter) {
  const int lane = threadIdx.x & 31;
  const int n = count_dev ? min(*count_dev, n_max) : n_max;
  for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += gridDim.x * (blockDim.x >> 5)) {
    const size_t row = (size_t)idx[i];
    const float4* s4 = reinterpret_cast<const float4*>(src + (scatter ? (size_t)i : row) * dim);
    float4* d4 = reinterpret_cast<float4*>(dst + (scatter ? row : (size_t)i) * dim);
    for (int c = lane; c < dim / 4; c += 32) d4[c] = s4[c];
  }
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
  dim3 grid(ceil_div(side, SS_K), ceil_div(tokens, SS_T));
  side_scores_kernel<<<grid, 256, 0, ctx->stream>>>(query, ld_query, 0, left_keys, left_scores, tokens, side, half);
  HL_LAUNCH_CHECK("side_scores_kernel");
  side_scores_kernel<<<grid, 256, 0, ctx->stream>>>(query, ld_query, half, right_keys, right_scores, tokens, side, half);
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
  if (side <= 512)
    product_key_topk_kernel<16><<<ceil_div(tokens, 4), 128, 0, ctx->stream>>>(left_scores, right_scores, out, tokens, side,
                                                                              top_k, beam, ctx->status_dev);
  else
    product_key_topk_kernel<PK_MAX_PER_LANE><<<ceil_div(tokens, 4), 128, 0, ctx->stream>>>(
        left_scores, right_scores, out, tokens, side, top_k, beam, ctx->status_dev);
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
  if (side > 0 && (grad_left_or_keys || grad_right_keys)) {
    const int half = key_dim / 2;
    const size_t smem = sizeof(float) * (size_t)DK_TOKENS * (DK_ROWS + DK_COLS);
    const int col_blocks = ceil_div(half, DK_COLS), row_blocks = ceil_div(side, DK_ROWS);
    const int token_blocks =
        std::max(1, std::min(ceil_div(tokens, 64), std::max(1, (2 * ctx->sm_count) / (2 * col_blocks * row_blocks))));
    const int tokens_per_block = ceil_div(tokens, token_blocks);
    rc = ensure_workspace(ctx, sizeof(float) * (size_t)token_blocks * 2 * side * half);
    if (rc != HL_OK) return rc;
    float* partial = reinterpret_cast<float*>(ctx->workspace);
    HL_CUDA(cudaFuncSetAttribute(product_key_dkeys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    product_key_dkeys_kernel<<<dim3(token_blocks, col_blocks * row_blocks, 2), 256, smem, ctx->stream>>>(
        indices, query, ld_query, grad_scores, partial, tokens, top_k, side, half, slots, tokens_per_block, col_blocks);
    HL_LAUNCH_CHECK("product_key_dkeys_kernel");
    const size_t total = 2 * (size_t)side * half;
    fold_key_partials_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(partial, grad_left_or_keys, grad_right_keys,
                                                                                       token_blocks, side, half);
    HL_LAUNCH_CHECK("fold_key_partials_kernel");
    count_launch(ctx, 2);
  }
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

}  // extern "C" (reopened below)

namespace hl {
// Stream-explicit forms, used by the data-parallel row exchange on the collective stream.
int mark_rows_on(hl_ctx* ctx, cudaStream_t stream, const int64_t* selected_rows, long long n_selected, const unsigned char* row_mask,
                 unsigned char* flags, int rows) {
  if (n_selected <= 0) return HL_OK;
  mark_rows_kernel<<<(unsigned)ceil_div_ll(n_selected, 256), 256, 0, stream>>>(selected_rows, n_selected, flags, row_mask, rows,
                                                                             ctx->status_dev);
  HL_LAUNCH_CHECK("mark_rows_kernel");
  count_launch(ctx);
  return HL_OK;
}
int mask_to_indices_on(hl_ctx* ctx, cudaStream_t stream, const unsigned char* mask, int rows, int64_t* out, int* count_dev) {
  mask_to_indices_kernel<<<1, 1024, 0, stream>>>(mask, rows, out, count_dev);
  HL_LAUNCH_CHECK("mask_to_indices_kernel");
  count_launch(ctx);
  return HL_OK;
}
int move_rows_on(hl_ctx* ctx, cudaStream_t stream, const float* src, const int64_t* idx, const int* count_dev, int n_max, int dim,
                 float* dst, bool scatter) {
  if (n_max <= 0) return HL_OK;
  const int blocks = std::min(ceil_div(n_max, 8), ctx->sm_count * 8);
  move_rows_kernel<<<blocks, 256, 0, stream>>>(src, idx, count_dev, n_max, dim, dst, scatter ? 1 : 0);
  HL_LAUNCH_CHECK("move_rows_kernel");
  count_launch(ctx);
  return HL_OK;
}
}  // namespace hl

extern "C" {

int hl_mark_rows_u8(hl_ctx* ctx, const int64_t* selected_rows, long long n_selected, const unsigned char* row_mask,
                    unsigned char* flags, int rows) {
  HL_REQUIRE(ctx && selected_rows && flags, "hl_mark_rows_u8: null argument");
  HL_REQUIRE(rows > 0, "hl_mark_rows_u8: requires non-zero rows");
  return mark_rows_on(ctx, ctx->stream, selected_rows, n_selected, row_mask, flags, rows);
}

int hl_mask_to_indices_u8(hl_ctx* ctx, const unsigned char* mask, int rows, int64_t* out_indices, int* count_dev) {
  HL_REQUIRE(ctx && mask && out_indices && count_dev, "hl_mask_to_indices_u8: null argument");
  HL_REQUIRE(rows > 0, "hl_mask_to_indices_u8: requires non-zero rows");
  return mask_to_indices_on(ctx, ctx->stream, mask, rows, out_indices, count_dev);
}

int hl_gather_rows_f32(hl_ctx* ctx, const float* src, const int64_t* indices, int n, int dim, float* dst) {
  HL_REQUIRE(ctx && src && indices && dst, "hl_gather_rows_f32: null argument");
  HL_REQUIRE(n >= 0 && dim > 0 && dim % 4 == 0, "hl_gather_rows_f32: row_dim must be a positive multiple of 4");
  return move_rows_on(ctx, ctx->stream, src, indices, nullptr, n, dim, dst, false);
}

int hl_scatter_rows_f32(hl_ctx* ctx, const float* src, const int64_t* indices, int n, int dim, float* dst) {
  HL_REQUIRE(ctx && src && indices && dst, "hl_scatter_rows_f32: null argument");
  HL_REQUIRE(n >= 0 && dim > 0 && dim % 4 == 0, "hl_scatter_rows_f32: row_dim must be a positive multiple of 4");
  return move_rows_on(ctx, ctx->stream, src, indices, nullptr, n, dim, dst, true);
}

int hl_sparse_rows_sum_squares_f32(hl_ctx* ctx, const float* grad, const int64_t* selected_rows, long long n_selected,
                                   const unsigned char* row_mask, unsigned char* row_flags, int rows, int row_dim,
                                   double* sum_dev) {
  HL_REQUIRE(ctx && grad && selected_rows && row_flags && sum_dev, "hl_sparse_rows_sum_squares_f32: null argument");
  HL_REQUIRE(rows > 0 && row_dim > 0, "hl_sparse_rows_sum_squares_f32: requires non-zero rows/row_dim");
  if (n_selected <= 0) return HL_OK;
  mark_rows_kernel<<<(unsigned)ceil_div_ll(n_selected, 256), 256, 0, ctx->stream>>>(selected_rows, n_selected, row_flags,
                                                                                  row_mask, rows, ctx->status_dev);
  HL_LAUNCH_CHECK("mark_rows_kernel");
  flagged_rows_sum_squares_kernel<<<ceil_div(rows, 8), 256, 0, ctx->stream>>>(grad, row_flags, rows, row_dim, sum_dev);
  HL_LAUNCH_CHECK("flagged_rows_sum_squares_kernel");
  count_launch(ctx, 2);
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
