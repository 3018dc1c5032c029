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
  // 16-byte loads need four-element granularity everywhere an address is formed
  const bool vec = (half_dim % 4) == 0 && (ld_q % 4) == 0 && (q_off % 4) == 0 &&
                   ((reinterpret_cast<uintptr_t>(query) | reinterpret_cast<uintptr_t>(keys)) & 15) == 0;
  for (int j0 = 0; j0 < half_dim; j0 += SS_J) {
    // stage the slice transposed.  Consecutive threads take consecutive rows, so the shared-memory stores of a warp
    // fall into 32 different banks; each thread brings four consecutive j of its row with one 16-byte load.
    if (vec) {
      for (int i = threadIdx.x; i < SS_T * (SS_J / 4); i += 256) {
        const int t = i % SS_T, j = (i / SS_T) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t0 + t < tokens && j0 + j < half_dim)
          x = *reinterpret_cast<const float4*>(query + (size_t)(t0 + t) * ld_q + q_off + j0 + j);
        sq[j][t] = x.x; sq[j + 1][t] = x.y; sq[j + 2][t] = x.z; sq[j + 3][t] = x.w;
      }
      for (int i = threadIdx.x; i < SS_K * (SS_J / 4); i += 256) {
        const int kk = i % SS_K, j = (i / SS_K) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k0 + kk < side && j0 + j < half_dim)
          x = __ldg(reinterpret_cast<const float4*>(keys + (size_t)(k0 + kk) * half_dim + j0 + j));
        sk[j][kk] = x.x; sk[j + 1][kk] = x.y; sk[j + 2][kk] = x.z; sk[j + 3][kk] = x.w;
      }
    } else {
      for (int i = threadIdx.x; i < SS_T * SS_J; i += 256) {
        const int t = i % SS_T, j = i / SS_T;
        sq[j][t] = (t0 + t < tokens && j0 + j < half_dim) ? query[(size_t)(t0 + t) * ld_q + q_off + j0 + j] : 0.f;
      }
      for (int i = threadIdx.x; i < SS_K * SS_J; i += 256) {
        const int kk = i % SS_K, j = i / SS_K;
        sk[j][kk] = (k0 + kk < side && j0 + j < half_dim) ? keys[(size_t)(k0 + kk) * half_dim + j0 + j] : 0.f;
      }
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
// (desc sum, asc slot).  One warp per token; side <= 2048, beam <= 32, top_k <= beam*beam.
//
// The selection never walks the side scores one winner at a time.  Scores become order-preserving 32-bit keys held
// in registers; the beam-th largest key is found by a four-pass radix select over a per-warp histogram; the chosen
// entries are compacted in index order (which settles ties at the threshold), sorted across the lanes, and the
// final top-k merges the 32 sorted rows `left[i] + right[.]` with one pointer per lane: a round is two warp
// reductions, and only the winning lane advances. ---------------------------------------------------------------
constexpr int PK_MAX_PER_LANE = 64;

// a > b as floats  <=>  okey(a) > okey(b); both zeros share a key, a NaN gets the lowest key 1, 0 means "no entry"
__device__ __forceinline__ unsigned okey(float f) {
  if (f != f) return 1u;
  const unsigned u = __float_as_uint(f == 0.f ? 0.f : f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float okey_value(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

template <int PER_LANE>
__global__ void __launch_bounds__(128)
product_key_topk_kernel(const float* __restrict__ left, const float* __restrict__ right, int64_t* __restrict__ out,
                        int tokens, int side, int top_k, int beam, int* __restrict__ status) {
  __shared__ unsigned s_hist[4][256];
  __shared__ unsigned s_key[4][32];
  __shared__ int s_index[4][32];
  __shared__ float s_rscore[4][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int token = blockIdx.x * 4 + w;
  if (token >= tokens) return;
  const unsigned full = 0xffffffffu, below = (1u << lane) - 1u;
  unsigned l_key = 0u;  // left beam entry `lane` after the sort
  int l_idx = 0;
  for (int sd = 0; sd < 2; ++sd) {
    const float* s = (sd == 0 ? left : right) + (size_t)token * side;
    unsigned key[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) key[i] = (i * 32 + lane < side) ? okey(s[i * 32 + lane]) : 0u;
    // radix select, 8 bits a pass from the top: afterwards `kstar` is the beam-th largest key and `need` says how
    // many entries equal to it belong to the beam
    unsigned kstar = 0u, decided = 0u;
    int need = beam;
#pragma unroll 1
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = lane; b < 256; b += 32) s_hist[w][b] = 0u;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (key[i] != 0u && (key[i] & decided) == kstar) atomicAdd(&s_hist[w][(key[i] >> shift) & 255u], 1u);
      __syncwarp();
      unsigned c[8], mine = 0u;  // the lane owns digits 8*lane .. 8*lane+7
#pragma unroll
      for (int b = 0; b < 8; ++b) { c[b] = s_hist[w][lane * 8 + b]; mine += c[b]; }
      unsigned from_here = mine;  // entries whose digit is in this lane's range or above
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned y = __shfl_down_sync(full, from_here, o);
        if (lane + o < 32) from_here += y;
      }
      const unsigned above = from_here - mine;
      const bool here = above < (unsigned)need && from_here >= (unsigned)need;
      int digit = 0;
      unsigned over = 0u;
      if (here) {
        unsigned run = above;
        bool found = false;
#pragma unroll
        for (int b = 7; b >= 0; --b) {
          if (!found) {
            if (run + c[b] >= (unsigned)need) { digit = lane * 8 + b; over = run; found = true; }
            else run += c[b];
          }
        }
      }
      const unsigned who = __ballot_sync(full, here);
      const int src = who ? __ffs(who) - 1 : 0;  // who == 0 only with fewer than `beam` entries, which the host rejects
      digit = __shfl_sync(full, digit, src);
      over = __shfl_sync(full, over, src);
      kstar |= (unsigned)digit << shift;
      decided |= 255u << shift;
      need -= (int)over;
      __syncwarp();
    }
    // compaction in index order: everything above the threshold, and the first `need` entries equal to it
    int base = 0, eq_seen = 0;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const bool eq = key[i] == kstar && kstar != 0u;
      const unsigned b_eq = __ballot_sync(full, eq);
      const bool take = (key[i] > kstar && kstar != 0u) || (eq && eq_seen + __popc(b_eq & below) < need);
      eq_seen += __popc(b_eq);
      const unsigned b_take = __ballot_sync(full, take);
      if (take) {
        const int pos = base + __popc(b_take & below);
        if (pos < 32) { s_key[w][pos] = key[i]; s_index[w][pos] = i * 32 + lane; }
      }
      base += __popc(b_take);
    }
    __syncwarp();
    // sort the beam across the lanes: key descending, index ascending
    const bool valid = lane < base && lane < 32;
    unsigned long long c64 = valid ? ((unsigned long long)s_key[w][lane] << 32) | (0xffffffffu - (unsigned)s_index[w][lane]) : 0ull;
#pragma unroll
    for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        const unsigned long long other = __shfl_xor_sync(full, c64, stride);
        const bool keep_max = ((lane & stride) == 0) == ((lane & size) == 0);
        c64 = keep_max ? (c64 > other ? c64 : other) : (c64 < other ? c64 : other);
      }
    }
    const unsigned k_sorted = (unsigned)(c64 >> 32);
    const int i_sorted = (int)(0xffffffffu - (unsigned)(c64 & 0xffffffffull));
    __syncwarp();
    if (sd == 0) {
      l_key = k_sorted;
      l_idx = i_sorted;
    } else {
      s_key[w][lane] = k_sorted;
      s_index[w][lane] = i_sorted;
      s_rscore[w][lane] = okey_value(k_sorted);
    }
    __syncwarp();
  }
  // row `lane` of the candidate matrix: left[lane] + right[j], non-increasing in j because the right beam is sorted
  // and f32 addition is monotone.  Equal sums sit next to each other; among them the lowest slot goes first.
  const bool has = lane < beam && l_key != 0u;
  const float ls = okey_value(l_key);
  const unsigned beam_mask = beam >= 32 ? 0xffffffffu : ((1u << beam) - 1u);
  unsigned used = 0u;
  unsigned head_key = 0u, head_slot = 0xffffffffu;
  int head_j = 0;
  auto advance = [&]() {
    head_key = 0u;
    head_slot = 0xffffffffu;
    const unsigned avail = ~used & beam_mask;
    if (!has || avail == 0u) return;
    const int j = __ffs(avail) - 1;
    if (s_key[w][j] == 0u) return;
    const float sum = __fadd_rn(ls, s_rscore[w][j]);
    int best_ri = s_index[w][j], best_j = j;
    for (int jj = j + 1; jj < beam; ++jj) {
      if (s_key[w][jj] == 0u || !(__fadd_rn(ls, s_rscore[w][jj]) == sum)) break;
      if (!((used >> jj) & 1u) && s_index[w][jj] < best_ri) { best_ri = s_index[w][jj]; best_j = jj; }
    }
    head_key = okey(sum);
    head_slot = (unsigned)(l_idx * side + best_ri);
    head_j = best_j;
  };
  advance();
  for (int r = 0; r < top_k; ++r) {
    const unsigned m = __reduce_max_sync(full, head_key);
    if (m == 0u) {
      if (lane == 0) { atomicExch(status + ST_BAD_ARGUMENT, 1); out[(size_t)token * top_k + r] = 0; }
      continue;
    }
    const unsigned bs = __reduce_min_sync(full, head_key == m ? head_slot : 0xffffffffu);
    if (head_key == m && head_slot == bs) {  // slots differ between lanes: exactly one winner
      used |= 1u << head_j;
      advance();
    }
    if (lane == 0) out[(size_t)token * top_k + r] = (long long)bs;
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
  if (side > 0 && half % 4 == 0 && key_dim <= 1024 && (ld_q % 4) == 0 &&
      ((reinterpret_cast<uintptr_t>(query) | reinterpret_cast<uintptr_t>(left) | reinterpret_cast<uintptr_t>(right)) & 15) == 0) {
    // product-key form: the query sits in registers (a lane owns up to 8 four-column groups); slots are split into
    // their half-table rows once per 32 and handed around by shuffles; 32 per-lane partial dots are then summed
    // across the warp by a transposing butterfly (31 exchanges instead of 32 five-step reductions).
    const int groups = key_dim / 4, half_groups = half / 4;
    float4 qv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int gi = u * 32 + lane;
      qv[u] = gi < groups ? *reinterpret_cast<const float4*>(q + gi * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int k0 = 0; k0 < top_k; k0 += 32) {
      int my_li = -1, my_ri = 0;
      if (k0 + lane < top_k) {
        const long long slot = idx[(size_t)token * top_k + k0 + lane];
        if (slot >= 0 && slot < slots) {
          my_li = (int)((unsigned)slot / (unsigned)side);
          my_ri = (int)((unsigned)slot % (unsigned)side);
        } else {
          atomicExch(status + ST_BAD_INDEX, 1);
        }
      }
      double part[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const int li = __shfl_sync(0xffffffffu, my_li, k);
        const int ri = __shfl_sync(0xffffffffu, my_ri, k);
        // a lane's share (at most 32 products) is summed in f32, the 32 shares in f64: f64 multiply-adds run at a
        // fraction of the f32 rate and were the busiest pipe of this kernel
        float acc = 0.f;
        if (li >= 0) {
          const float4* lrow = reinterpret_cast<const float4*>(left + (size_t)li * half);
          const float4* rrow = reinterpret_cast<const float4*>(right + (size_t)ri * half);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int gi = u * 32 + lane;
            if (gi < groups) {
              const float4 kv = gi < half_groups ? __ldg(lrow + gi) : __ldg(rrow + (gi - half_groups));
              acc = fmaf(qv[u].x, kv.x, acc); acc = fmaf(qv[u].y, kv.y, acc);
              acc = fmaf(qv[u].z, kv.z, acc); acc = fmaf(qv[u].w, kv.w, acc);
            }
          }
        }
        part[k] = (double)acc;
      }
      // after the step with distance d, a lane keeps the half of its values whose index has the same d-bit as the lane
#pragma unroll
      for (int d = 16; d >= 1; d >>= 1) {
        const bool upper = (lane & d) != 0;
#pragma unroll
        for (int i = 0; i < d; ++i) {
          const double send = upper ? part[i] : part[i + d];
          const double keep = upper ? part[i + d] : part[i];
          part[i] = keep + __shfl_xor_sync(0xffffffffu, send, d);
        }
      }
      if (k0 + lane < top_k) scores[(size_t)token * top_k + k0 + lane] = (float)part[0];
    }
    return;
  }
  for (int k = 0; k < top_k; ++k) {
    const long long slot = idx[(size_t)token * top_k + k];
    if (slot < 0 || slot >= slots) {
      if (lane == 0) { atomicExch(status + ST_BAD_INDEX, 1); scores[(size_t)token * top_k + k] = 0.f; }
      continue;
    }
    double acc = 0.0;
    if (side > 0) {
      const unsigned s32 = (unsigned)slot, side32 = (unsigned)side;
      const float* kl = left + (size_t)(s32 / side32) * half;
      const float* kr = right + (size_t)(s32 % side32) * half;
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
  if (dq) {
    if (side > 0 && half % 4 == 0 && key_dim <= 1024 && (ld_dq % 4) == 0 &&
        ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(left) | reinterpret_cast<uintptr_t>(right)) & 15) == 0) {
      // product-key form: a lane owns up to 8 four-column groups of the query gradient; slots and score gradients are
      // read once per 32 and handed around by shuffles, table rows come in with 16-byte loads
      float4 acc[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      const int groups = key_dim / 4, half_groups = half / 4;
      for (int k0 = 0; k0 < top_k; k0 += 32) {
        int my_li = -1, my_ri = 0;
        float my_g = 0.f;
        if (k0 + lane < top_k) {
          const long long slot = idx[(size_t)token * top_k + k0 + lane];
          if (slot >= 0 && slot < slots) {
            my_li = (int)((unsigned)slot / (unsigned)side);
            my_ri = (int)((unsigned)slot % (unsigned)side);
            my_g = grad_scores[(size_t)token * top_k + k0 + lane];
          }
        }
        const int n = min(32, top_k - k0);
        for (int k = 0; k < n; ++k) {
          const int li = __shfl_sync(0xffffffffu, my_li, k);
          const int ri = __shfl_sync(0xffffffffu, my_ri, k);
          const float g = __shfl_sync(0xffffffffu, my_g, k);
          if (li < 0) continue;
          const float4* lrow = reinterpret_cast<const float4*>(left + (size_t)li * half);
          const float4* rrow = reinterpret_cast<const float4*>(right + (size_t)ri * half);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int gi = u * 32 + lane;
            if (gi < groups) {
              const float4 kv = gi < half_groups ? __ldg(lrow + gi) : __ldg(rrow + (gi - half_groups));
              acc[u].x = fmaf(g, kv.x, acc[u].x); acc[u].y = fmaf(g, kv.y, acc[u].y);
              acc[u].z = fmaf(g, kv.z, acc[u].z); acc[u].w = fmaf(g, kv.w, acc[u].w);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int gi = u * 32 + lane;
        if (gi < groups) *reinterpret_cast<float4*>(dq + (size_t)token * ld_dq + gi * 4) = acc[u];
      }
    } else {
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
        dq[(size_t)token * ld_dq + j] = (float)acc;
      }
    }
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
// dK = Wᵀ·Q with W[t, row] = sum of the g[t,k] whose slot maps to `row`: a CTA owns a block of tokens, 256 rows
// and 64 columns of one table; per slice of 32 tokens it builds W in shared memory (one warp per token, its
// duplicates added in slot order), multiplies with an 8 x 8 register tile per thread (two CTAs per SM), and clears the entries it
// set.  The CTA's tile goes out as a partial result that fold_key_partials_kernel adds up in block order, so the
// result does not depend on scheduling.
constexpr int DK_COLS = 64;    // columns per CTA
constexpr int DK_ROWS = 256;   // table rows per CTA
constexpr int DK_TOKENS = 32;  // tokens per slice
__global__ void __launch_bounds__(256, 2)
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
  const int tr = threadIdx.x >> 3;  // 32 row groups of 8 rows
  const int tc = threadIdx.x & 7;   // 8 column groups of 8 columns
  float acc[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
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
    // W rows: warp w builds tokens w, w+8, ...  Each lane takes one selected slot; lanes whose slots share a table
    // row add their gradients one after the other in slot order (round r = the lane's rank among its duplicates),
    // so a row's sum is formed in the same order on every run.
    for (int t = warp; t < DK_TOKENS; t += 8) {
      if (t0 + t >= t_end) break;
      for (int k0 = 0; k0 < top_k; k0 += 32) {
        int row = -1;
        float g = 0.f;
        if (k0 + lane < top_k) {
          const long long slot = idx[(size_t)(t0 + t) * top_k + k0 + lane];
          if (slot >= 0 && slot < slots) {
            const unsigned s32 = (unsigned)slot, side32 = (unsigned)side;
            row = (int)(table ? s32 % side32 : s32 / side32) - r0;
            g = grad_scores[(size_t)(t0 + t) * top_k + k0 + lane];
            if (row < 0 || row >= DK_ROWS) row = -1;
          }
        }
        const unsigned same = __match_any_sync(0xffffffffu, row);
        const int rank = row < 0 ? -1 : __popc(same & ((1u << lane) - 1u));
        const int rounds = __reduce_max_sync(0xffffffffu, rank) + 1;
        for (int r = 0; r < rounds; ++r) {
          if (rank == r) w_tile[t * DK_ROWS + row] += g;
          __syncwarp();
        }
      }
    }
    __syncthreads();
    const int tn = min(DK_TOKENS, t_end - t0);
    for (int t = 0; t < tn; ++t) {
      float wv[8], qv[8];
#pragma unroll
      for (int a = 0; a < 8; a += 4) {
        const float4 x = *reinterpret_cast<const float4*>(&w_tile[t * DK_ROWS + tr * 8 + a]);
        wv[a] = x.x; wv[a + 1] = x.y; wv[a + 2] = x.z; wv[a + 3] = x.w;
      }
#pragma unroll
      for (int b = 0; b < 8; b += 4) {
        const float4 x = *reinterpret_cast<const float4*>(&q_tile[t * DK_COLS + tc * 8 + b]);
        qv[b] = x.x; qv[b + 1] = x.y; qv[b + 2] = x.z; qv[b + 3] = x.w;
      }
#pragma unroll
      for (int a = 0; a < 8; ++a)
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
        const unsigned s32 = (unsigned)slot, side32 = (unsigned)side;
        const int row = (int)(table ? s32 % side32 : s32 / side32) - r0;
        if (row >= 0 && row < DK_ROWS) w_tile[t * DK_ROWS + row] = 0.f;
      }
    }
  }
  // partial[block][table][side][half]
  float* dst = partial + ((size_t)blockIdx.x * 2 + table) * side * half;
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int row = r0 + tr * 8 + a;
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
  if (dim <= 1024) {
    // slots and weights are read once per 32 and handed around by shuffles; a lane owns up to 8 four-column groups and
    // sums its at most top_k products per column in f32 (f64 multiply-adds run at a fraction of the f32 rate)
    const int groups = dim / 4;
    float4 acc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < top_k; k0 += 32) {
      long long my_row = -1;
      float my_w = 0.f;
      if (k0 + lane < top_k) {
        my_row = idx[(size_t)token * top_k + k0 + lane];
        my_w = weights[(size_t)token * top_k + k0 + lane];
        if (my_row < 0 || my_row >= rows) { atomicExch(status + ST_BAD_INDEX, 1); my_row = -1; }
      }
      const int n = min(32, top_k - k0);
      for (int k = 0; k < n; ++k) {
        const long long r = __shfl_sync(0xffffffffu, my_row, k);
        const float w = __shfl_sync(0xffffffffu, my_w, k);
        if (r < 0) continue;
        const float4* row = reinterpret_cast<const float4*>(values + (size_t)r * dim);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int gi = u * 32 + lane;
          if (gi < groups) {
            const float4 v = __ldg(row + gi);
            acc[u].x = fmaf(w, v.x, acc[u].x); acc[u].y = fmaf(w, v.y, acc[u].y);
            acc[u].z = fmaf(w, v.z, acc[u].z); acc[u].w = fmaf(w, v.w, acc[u].w);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int gi = u * 32 + lane;
      if (gi < groups) reinterpret_cast<float4*>(out + (size_t)token * dim)[gi] = acc[u];
    }
    return;
  }
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

// ---- weighted value backward in row order ---------------------------------------------------------------------
// With many more (token, slot) events than distinct rows (about 26 events per row at the memory-transformer size),
// per-event 16-byte atomics pile onto hot rows in L2.  Events are therefore sorted by row (radix sort over as many key
// bits as the row count needs); a warp takes 32 consecutive sorted events, keeps the value row of the current run and
// the run's gradient sum in registers, and issues one set of atomics per run (and per chunk boundary).  The weight
// gradients, dot(grad_out[token], values[row]), come from the same pass: one 2 KB read of grad_out per event is all
// the traffic that does not stay in registers.
__global__ void value_event_keys_kernel(const int64_t* __restrict__ idx, long long n, int rows, int* __restrict__ keys,
                                        int* __restrict__ events, float* __restrict__ dweights, int* __restrict__ status) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long r = idx[i];
  const bool bad = r < 0 || r >= rows;
  keys[i] = bad ? rows : (int)r;  // out-of-range slots sort behind every row and are skipped by the row walk,
  events[i] = (int)i;
  if (bad) {                      // so they are reported and their weight gradient is written here
    atomicExch(status + ST_BAD_INDEX, 1);
    if (dweights) dweights[i] = 0.f;
  }
}

// ---- stable radix sort of (row key, event) pairs, eight bits a pass --------------------------------------------
// The row-ordered value backward needs the step's (token, slot) events grouped by table row, events of a row in
// ascending order (that order fixes the f32 summation order of a row's gradient).  Three kernels a pass:
// digit histograms per tile of 2048 keys, an exclusive scan of every digit's row of the digit-major histogram array
// (one block per digit; the scatter adds the scan over the 256 digit totals itself), and a scatter in which every
// warp walks its 256 keys in order, ranking equal digits with warp matches, so the sort is stable.
constexpr int RS_BITS = 8, RS_DIGITS = 1 << RS_BITS, RS_WARPS = 8, RS_THREADS = RS_WARPS * 32;
constexpr int RS_PER_WARP = 256, RS_TILE = RS_WARPS * RS_PER_WARP;

// Digit counts of each warp's keys in shared memory: lanes with equal digits are found with a warp match, the
// lowest of them adds the group's size.
__device__ __forceinline__ void rs_count_tile(const int* __restrict__ keys, long long n, int shift,
                                              int (*wc)[RS_DIGITS]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < RS_WARPS * RS_DIGITS; i += RS_THREADS) (&wc[0][0])[i] = 0;
  __syncthreads();
  const long long base = (long long)blockIdx.x * RS_TILE + (long long)warp * RS_PER_WARP;
  for (int r = 0; r < RS_PER_WARP / 32; ++r) {
    const long long i = base + r * 32 + lane;
    const bool in = i < n;
    const unsigned alive = __ballot_sync(0xffffffffu, in);
    if (in) {
      const int d = (keys[i] >> shift) & (RS_DIGITS - 1);
      const unsigned peers = __match_any_sync(alive, d);
      if (lane == __ffs(peers) - 1) wc[warp][d] += __popc(peers);
    }
    __syncwarp();
  }
  __syncthreads();
}

__global__ void __launch_bounds__(RS_THREADS)
radix_hist_kernel(const int* __restrict__ keys, long long n, int shift, int* __restrict__ hist, int n_tiles) {
  __shared__ int wc[RS_WARPS][RS_DIGITS];
  rs_count_tile(keys, n, shift, wc);
  for (int d = threadIdx.x; d < RS_DIGITS; d += RS_THREADS) {
    int t = 0;
#pragma unroll
    for (int w = 0; w < RS_WARPS; ++w) t += wc[w][d];
    hist[(size_t)d * n_tiles + blockIdx.x] = t;  // digit-major: a scan over the array gives every (digit, tile) its start
  }
}

// Block d scans row d of the digit-major histogram in place (exclusive) and writes the row's total.
__global__ void __launch_bounds__(RS_THREADS)
radix_scan_rows_kernel(int* __restrict__ hist, int n_tiles, int* __restrict__ totals) {
  __shared__ int warp_sums[RS_WARPS];
  __shared__ int carry;
  int* row = hist + (size_t)blockIdx.x * n_tiles;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n_tiles; base += RS_THREADS) {
    const int i = base + threadIdx.x;
    const int v = i < n_tiles ? row[i] : 0;
    int inc = v;  // inclusive scan within the warp
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += t;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
    if (i < n_tiles) row[i] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == RS_THREADS - 1) carry = before + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = carry;
}

__global__ void __launch_bounds__(RS_THREADS)
radix_scatter_kernel(const int* __restrict__ keys, const int* __restrict__ vals, int* __restrict__ keys_out,
                     int* __restrict__ vals_out, long long n, int shift, const int* __restrict__ starts,
                     const int* __restrict__ totals, int n_tiles) {
  __shared__ int wc[RS_WARPS][RS_DIGITS];  // counts, then the running output position of each (warp, digit)
  __shared__ int dbase[RS_DIGITS];         // keys with a smaller digit, over all tiles
  __shared__ int wsum[RS_WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  static_assert(RS_DIGITS == RS_THREADS, "one thread per digit");
  {
    const int v = totals[threadIdx.x];
    int inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += t;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    dbase[threadIdx.x] = before + inc - v;
  }
  rs_count_tile(keys, n, shift, wc);
  for (int d = threadIdx.x; d < RS_DIGITS; d += RS_THREADS) {
    int run = dbase[d] + starts[(size_t)d * n_tiles + blockIdx.x];
#pragma unroll
    for (int w = 0; w < RS_WARPS; ++w) {
      const int c = wc[w][d];
      wc[w][d] = run;
      run += c;
    }
  }
  __syncthreads();
  const long long base = (long long)blockIdx.x * RS_TILE + (long long)warp * RS_PER_WARP;
  for (int r = 0; r < RS_PER_WARP / 32; ++r) {
    const long long i = base + r * 32 + lane;
    const bool in = i < n;
    const unsigned alive = __ballot_sync(0xffffffffu, in);
    if (in) {
      const int key = keys[i];
      const int d = (key >> shift) & (RS_DIGITS - 1);
      const unsigned peers = __match_any_sync(alive, d);
      const int leader = __ffs(peers) - 1;
      int first = 0;
      if (lane == leader) {
        first = wc[warp][d];
        wc[warp][d] = first + __popc(peers);
      }
      first = __shfl_sync(peers, first, leader);
      const int pos = first + __popc(peers & ((1u << lane) - 1u));  // earlier lanes hold earlier keys
      keys_out[pos] = key;
      vals_out[pos] = vals[i];
    }
    __syncwarp();
  }
}

template <int VPL>  // 16-byte pieces of a row per lane: dim <= VPL * 128
__global__ void __launch_bounds__(128)
weighted_value_bwd_sorted_kernel(const int* __restrict__ keys, const int* __restrict__ events,
                                 const float* __restrict__ weights, const float* __restrict__ values,
                                 const float* __restrict__ grad_out, float* __restrict__ dweights,
                                 float* __restrict__ dvalues, long long n, int top_k, int rows, int dim) {
  const int lane = threadIdx.x & 31;
  const long long base = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 32;
  if (base >= n) return;
  const int groups = dim / 4;
  int my_key = rows, my_event = 0;
  float my_w = 0.f;
  if (base + lane < n) {
    my_key = keys[base + lane];
    my_event = events[base + lane];
    if (my_key < rows) my_w = weights[my_event];
  }
  float4 acc[VPL], vrow[VPL];
#pragma unroll
  for (int u = 0; u < VPL; ++u) acc[u] = vrow[u] = make_float4(0.f, 0.f, 0.f, 0.f);
  int cur = -1;
  auto flush = [&]() {
    if (cur < 0 || !dvalues) return;
#pragma unroll
    for (int u = 0; u < VPL; ++u) {
      const int gi = u * 32 + lane;
      if (gi < groups) atomicAdd(reinterpret_cast<float4*>(dvalues + (size_t)cur * dim) + gi, acc[u]);
      acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  for (int i = 0; i < 32; ++i) {
    const int key = __shfl_sync(0xffffffffu, my_key, i);
    if (key >= rows) break;  // sorted: nothing valid follows
    const int event = __shfl_sync(0xffffffffu, my_event, i);
    const float w = __shfl_sync(0xffffffffu, my_w, i);
    if (key != cur) {
      flush();
      cur = key;
      if (dweights) {
#pragma unroll
        for (int u = 0; u < VPL; ++u) {
          const int gi = u * 32 + lane;
          if (gi < groups) vrow[u] = __ldg(reinterpret_cast<const float4*>(values + (size_t)key * dim) + gi);
        }
      }
    }
    const float4* go = reinterpret_cast<const float4*>(grad_out + (size_t)(event / top_k) * dim);
    float share = 0.f;  // this lane's part of the dot product in f32, the 32 parts are summed in f64
#pragma unroll
    for (int u = 0; u < VPL; ++u) {
      const int gi = u * 32 + lane;
      if (gi < groups) {
        const float4 g = __ldg(go + gi);
        share = fmaf(g.x, vrow[u].x, share); share = fmaf(g.y, vrow[u].y, share);
        share = fmaf(g.z, vrow[u].z, share); share = fmaf(g.w, vrow[u].w, share);
        acc[u].x = fmaf(w, g.x, acc[u].x); acc[u].y = fmaf(w, g.y, acc[u].y);
        acc[u].z = fmaf(w, g.z, acc[u].z); acc[u].w = fmaf(w, g.w, acc[u].w);
      }
    }
    if (dweights) {
      const double dot = warp_sum((double)share);
      if (lane == 0) dweights[event] = (float)dot;
    }
  }
  flush();
}

// ---- access counts: counts[r] += occurrences of r among the selected rows (kernels.ptx:813-886) ---------------
__global__ void access_count_rows_kernel(const int64_t* __restrict__ selected, long long n, int rows,
                                         unsigned long long* __restrict__ counts, int* __restrict__ status) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long r = selected[i];
    if (r < 0 || r >= rows) { atomicExch(status + ST_BAD_INDEX, 1); continue; }
    atomicAdd(counts + r, 1ull);
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
  const long long n = (long long)tokens * top_k;
  if (grad_values && n >= 32768 && n < (1ll << 31) - 64 && dim <= 1024 && rows < (1 << 30)) {
    // row order (see weighted_value_bwd_sorted_kernel).  Scratch: keys and events in and out, and the sort's own space.
    int end_bit = 1;
    while ((1ll << end_bit) <= rows) ++end_bit;  // the sentinel key `rows` must sort last
    const int n_tiles = (int)ceil_div_ll(n, RS_TILE);
    const size_t arr = ((size_t)n * sizeof(int) + 255) & ~size_t(255);
    const size_t hist_bytes = ((size_t)RS_DIGITS * (n_tiles + 1) * sizeof(int) + 255) & ~size_t(255);  // rows, then totals
    rc = ensure_workspace(ctx, 4 * arr + hist_bytes);
    if (rc != HL_OK) return rc;
    uint8_t* ws = reinterpret_cast<uint8_t*>(ctx->workspace);
    int *keys_a = reinterpret_cast<int*>(ws), *ev_a = reinterpret_cast<int*>(ws + arr);
    int *keys_b = reinterpret_cast<int*>(ws + 2 * arr), *ev_b = reinterpret_cast<int*>(ws + 3 * arr);
    int* hist = reinterpret_cast<int*>(ws + 4 * arr);
    value_event_keys_kernel<<<(unsigned)ceil_div_ll(n, 256), 256, 0, ctx->stream>>>(indices, n, rows, keys_a, ev_a, grad_weights,
                                                                                     ctx->status_dev);
    HL_LAUNCH_CHECK("value_event_keys_kernel");
    int passes = 0;
    for (int shift = 0; shift < end_bit; shift += RS_BITS, ++passes) {
      radix_hist_kernel<<<n_tiles, RS_THREADS, 0, ctx->stream>>>(keys_a, n, shift, hist, n_tiles);
      HL_LAUNCH_CHECK("radix_hist_kernel");
      int* totals = hist + (size_t)RS_DIGITS * n_tiles;
      radix_scan_rows_kernel<<<RS_DIGITS, RS_THREADS, 0, ctx->stream>>>(hist, n_tiles, totals);
      HL_LAUNCH_CHECK("radix_scan_rows_kernel");
      radix_scatter_kernel<<<n_tiles, RS_THREADS, 0, ctx->stream>>>(keys_a, ev_a, keys_b, ev_b, n, shift, hist, totals, n_tiles);
      HL_LAUNCH_CHECK("radix_scatter_kernel");
      std::swap(keys_a, keys_b);
      std::swap(ev_a, ev_b);
    }
    const int *keys = keys_a, *ev = ev_a;  // the last pass's output
    count_launch(ctx, 3 * passes);
    const unsigned blocks = (unsigned)ceil_div_ll(ceil_div_ll(n, 32), 4);
    if (dim <= 512)
      weighted_value_bwd_sorted_kernel<4><<<blocks, 128, 0, ctx->stream>>>(keys, ev, weights, values, grad_out, grad_weights,
                                                                           grad_values, n, top_k, rows, dim);
    else
      weighted_value_bwd_sorted_kernel<8><<<blocks, 128, 0, ctx->stream>>>(keys, ev, weights, values, grad_out, grad_weights,
                                                                           grad_values, n, top_k, rows, dim);
    HL_LAUNCH_CHECK("weighted_value_bwd_sorted_kernel");
    count_launch(ctx, 2);
    return HL_OK;
  }
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

int hl_memory_access_count_rows_i64_u64(hl_ctx* ctx, const int64_t* selected_rows, long long n_selected, int slots,
                                        unsigned long long* counts) {
  HL_REQUIRE(ctx && counts, "hl_memory_access_count_rows_i64_u64: null argument");
  HL_REQUIRE(slots > 0, "memory_access_count_rows_i64_u64 requires non-zero memory_slots");
  HL_REQUIRE(n_selected >= 0 && (n_selected == 0 || selected_rows), "hl_memory_access_count_rows_i64_u64: null selected rows");
  if (n_selected == 0) return HL_OK;
  const unsigned blocks = (unsigned)std::min<long long>(ceil_div_ll(n_selected, 256), (long long)ctx->sm_count * 16);
  access_count_rows_kernel<<<blocks, 256, 0, ctx->stream>>>(selected_rows, n_selected, slots, counts, ctx->status_dev);
  HL_LAUNCH_CHECK("access_count_rows_kernel");
  count_launch(ctx);
  return HL_OK;
}

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
