// Layer norm, embedding gather / scatter-add and softmax cross-entropy with fused logits
// gradient.  Warp-per-row with shuffle reductions and 128-bit accesses; the reference's
// kernels are one thread per element with per-element row re-reduction (layer norm,
// heirloom-kernels/src/ptx/kernels.ptx:3296-3322) or a single thread for the whole loss
// (heirloom-kernels/src/cuda.rs:10328-10339).
#include "kernels.h"

namespace hl {
namespace {

// ---- vector access helpers ------------------------------------------------------------------
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 4;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
  }
};
template <typename T> __device__ __forceinline__ float load1(const T* p);
template <> __device__ __forceinline__ float load1<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) { return from_bf16(*p); }
template <typename T> __device__ __forceinline__ void store1(T* p, float v);
template <> __device__ __forceinline__ void store1<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = to_bf16(v); }

// ---- layer norm forward ---------------------------------------------------------------------
// One warp per row.  VEC4: features % 4 == 0 and every row start is vector aligned.
template <typename XT, typename YT, typename Acc, bool VEC4>
__global__ void layer_norm_fwd_kernel(const XT* __restrict__ x, const float* __restrict__ gamma,
                                      const float* __restrict__ beta, YT* __restrict__ y, float* __restrict__ mean_out,
                                      float* __restrict__ rstd_out, int rows, int features, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const XT* xr = x + (size_t)row * features;
  YT* yr = y + (size_t)row * features;
  Acc sum = 0;
  if (VEC4) {
    for (int c = lane * 4; c < features; c += 128) {
      float v[4];
      Vec<XT>::load(xr + c, v);
      sum += (Acc)v[0] + (Acc)v[1] + (Acc)v[2] + (Acc)v[3];
    }
  } else {
    for (int c = lane; c < features; c += 32) sum += (Acc)load1(xr + c);
  }
  const Acc mean = warp_sum(sum) / (Acc)features;
  Acc sq = 0;
  if (VEC4) {
    for (int c = lane * 4; c < features; c += 128) {
      float v[4];
      Vec<XT>::load(xr + c, v);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const Acc d = (Acc)v[i] - mean; sq += d * d; }
    }
  } else {
    for (int c = lane; c < features; c += 32) { const Acc d = (Acc)load1(xr + c) - mean; sq += d * d; }
  }
  const Acc var = warp_sum(sq) / (Acc)features;
  const Acc rstd = (Acc)1 / sqrt(var + (Acc)eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = (float)mean;
    if (rstd_out) rstd_out[row] = (float)rstd;
  }
  if (VEC4) {
    for (int c = lane * 4; c < features; c += 128) {
      float v[4], g[4], b[4], o[4];
      Vec<XT>::load(xr + c, v);
      Vec<float>::load(gamma + c, g);
      Vec<float>::load(beta + c, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = (float)(((Acc)v[i] - mean) * rstd * (Acc)g[i] + (Acc)b[i]);
      Vec<YT>::store(yr + c, o);
    }
  } else {
    for (int c = lane; c < features; c += 32)
      store1(yr + c, (float)(((Acc)load1(xr + c) - mean) * rstd * (Acc)gamma[c] + (Acc)beta[c]));
  }
}

// ---- layer norm backward --------------------------------------------------------------------
// Each warp walks rows of its block's slab.  Per row: two shuffle reductions, dx written, and
// the lane's own columns of dgamma/dbeta accumulated in registers (columns (j*32+lane)*4+e,
// j < 8, so features <= 1024).  Warps are then folded through shared memory into one partial
// row per block; a second kernel folds the partial rows in a fixed order.
constexpr int LNB_WARPS = 8;
constexpr int LNB_MAXJ = 8;

template <typename XT, typename Acc>
__global__ void __launch_bounds__(LNB_WARPS * 32)
layer_norm_bwd_kernel(const XT* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ dy,
                      const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                      const float* __restrict__ residual_grad, float* __restrict__ dx_f32,
                      __nv_bfloat16* __restrict__ dx_bf16, float* __restrict__ partial /*[blocks][2][features]*/,
                      int rows, int features, int rows_per_block, float eps) {
  extern __shared__ float lnb_smem[];  // [LNB_WARPS][2][features]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = blockIdx.x * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  Acc dg[LNB_MAXJ][4], db[LNB_MAXJ][4];
#pragma unroll
  for (int j = 0; j < LNB_MAXJ; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) { dg[j][e] = 0; db[j][e] = 0; }

  for (int row = r0 + warp; row < r1; row += LNB_WARPS) {
    const XT* xr = x + (size_t)row * features;
    const float* dyr = dy + (size_t)row * features;
    Acc mean, rstd;
    if (mean_in && rstd_in) {
      mean = (Acc)mean_in[row];
      rstd = (Acc)rstd_in[row];
    } else {
      Acc s = 0;
      for (int c = lane * 4; c < features; c += 128) {
        float v[4]; Vec<XT>::load(xr + c, v);
        s += (Acc)v[0] + (Acc)v[1] + (Acc)v[2] + (Acc)v[3];
      }
      mean = warp_sum(s) / (Acc)features;
      Acc q = 0;
      for (int c = lane * 4; c < features; c += 128) {
        float v[4]; Vec<XT>::load(xr + c, v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const Acc d = (Acc)v[i] - mean; q += d * d; }
      }
      rstd = (Acc)1 / sqrt(warp_sum(q) / (Acc)features + (Acc)eps);
    }
    Acc s1 = 0, s2 = 0;
#pragma unroll
    for (int j = 0; j < LNB_MAXJ; ++j) {
      const int c = (j * 32 + lane) * 4;
      if (c < features) {
        float v[4], g[4], d[4];
        Vec<XT>::load(xr + c, v);
        Vec<float>::load(gamma + c, g);
        Vec<float>::load(dyr + c, d);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const Acc xhat = ((Acc)v[e] - mean) * rstd;
          const Acc dxhat = (Acc)d[e] * (Acc)g[e];
          s1 += dxhat;
          s2 += dxhat * xhat;
          dg[j][e] += (Acc)d[e] * xhat;
          db[j][e] += (Acc)d[e];
        }
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
#pragma unroll
    for (int j = 0; j < LNB_MAXJ; ++j) {
      const int c = (j * 32 + lane) * 4;
      if (c < features) {
        float v[4], g[4], d[4], o[4];
        Vec<XT>::load(xr + c, v);
        Vec<float>::load(gamma + c, g);
        Vec<float>::load(dyr + c, d);
        float rg[4] = {0.f, 0.f, 0.f, 0.f};
        if (residual_grad) Vec<float>::load(residual_grad + (size_t)row * features + c, rg);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const Acc xhat = ((Acc)v[e] - mean) * rstd;
          const Acc dxhat = (Acc)d[e] * (Acc)g[e];
          const Acc dxv = rstd * ((Acc)features * dxhat - s1 - xhat * s2) / (Acc)features;
          o[e] = residual_grad ? (float)((Acc)rg[e] + (Acc)(float)dxv) : (float)dxv;
        }
        if (dx_f32) Vec<float>::store(dx_f32 + (size_t)row * features + c, o);
        if (dx_bf16) Vec<__nv_bfloat16>::store(dx_bf16 + (size_t)row * features + c, o);
      }
    }
  }
  // fold the warps
  float* mine = lnb_smem + (size_t)warp * 2 * features;
#pragma unroll
  for (int j = 0; j < LNB_MAXJ; ++j) {
    const int c = (j * 32 + lane) * 4;
    if (c < features) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mine[c + e] = (float)dg[j][e];
        mine[features + c + e] = (float)db[j][e];
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * features; c += blockDim.x) {
    Acc s = 0;
#pragma unroll
    for (int w = 0; w < LNB_WARPS; ++w) s += (Acc)lnb_smem[(size_t)w * 2 * features + c];
    partial[(size_t)blockIdx.x * 2 * features + c] = (float)s;
  }
}

__global__ void layer_norm_bwd_fold_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                           float* __restrict__ dbeta, int features, int blocks) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= 2 * features) return;
  double s = 0.0;
  for (int b = 0; b < blocks; ++b) s += (double)partial[(size_t)b * 2 * features + c];
  if (c < features) { if (dgamma) dgamma[c] = (float)s; }
  else if (dbeta) dbeta[c - features] = (float)s;
}

// ---- embedding ------------------------------------------------------------------------------
template <typename OT>
__global__ void embedding_fwd_kernel(const float* __restrict__ table, int table_rows, const int64_t* __restrict__ idx,
                                     const float* __restrict__ pos_table, int period, OT* __restrict__ out, int n,
                                     int dim, bool round_terms, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const long long id = idx[row];
  if (id < 0 || id >= table_rows) {
    if (lane == 0) atomicExch(status + ST_BAD_INDEX, 1);
    return;
  }
  const float* src = table + (size_t)id * dim;
  const float* pos = pos_table ? pos_table + (size_t)(row % period) * dim : nullptr;
  OT* dst = out + (size_t)row * dim;
  if ((dim & 3) == 0) {
    for (int c = lane * 4; c < dim; c += 128) {
      float v[4];
      Vec<float>::load(src + c, v);
      if (pos) {
        float pv[4];
        Vec<float>::load(pos + c, pv);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = round_terms ? bf16_round(v[e]) + bf16_round(pv[e]) : v[e] + pv[e];
      }
      Vec<OT>::store(dst + c, v);
    }
  } else {
    for (int c = lane; c < dim; c += 32) {
      float v = src[c];
      if (pos) v = round_terms ? bf16_round(v) + bf16_round(pos[c]) : v + pos[c];
      store1(dst + c, v);
    }
  }
}

__global__ void embedding_bwd_kernel(const float* __restrict__ grad_out, const int64_t* __restrict__ idx,
                                     float* __restrict__ grad_table, int table_rows, int n, int dim,
                                     int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const long long id = idx[row];
  if (id < 0 || id >= table_rows) {
    if (lane == 0) atomicExch(status + ST_BAD_INDEX, 1);
    return;
  }
  const float* src = grad_out + (size_t)row * dim;
  float* dst = grad_table + (size_t)id * dim;
  if ((dim & 3) == 0) {
    for (int c = lane * 4; c < dim; c += 128) {
      const float4 v = *reinterpret_cast<const float4*>(src + c);
      atomicAdd(reinterpret_cast<float4*>(dst + c), v);
    }
  } else {
    for (int c = lane; c < dim; c += 32) atomicAdd(dst + c, src[c]);
  }
}

// Position table gradient: rows n with the same n % period are summed in increasing n, so the
// result does not depend on scheduling.
__global__ void position_grad_kernel(const float* __restrict__ grad_out, float* __restrict__ pos_grad, int period,
                                     int n, int dim) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)period * dim) return;
  const int t = (int)(i / dim), c = (int)(i % dim);
  double s = 0.0;
  for (int r = t; r < n; r += period) s += (double)grad_out[(size_t)r * dim + c];
  pos_grad[i] += (float)s;
}

// ---- cross-entropy --------------------------------------------------------------------------
// One block per row.  Pass 1: online max / sum of exponentials; pass 2 (row still in L2):
// dlogits = (softmax - onehot) * scale.  Acc = double for the f32 parity route.
template <typename Acc, typename DT>
__global__ void cross_entropy_kernel(const float* __restrict__ logits, long long ld, const int64_t* __restrict__ targets,
                                     int rows, int classes, float scale, float* __restrict__ row_loss,
                                     DT* __restrict__ dlogits, long long ld_d, int* __restrict__ status) {
  __shared__ Acc sm[32];
  const int row = blockIdx.x;
  const float* z = logits + (size_t)row * ld;
  const long long target = targets[row];
  if (target < 0 || target >= classes) {
    if (threadIdx.x == 0) { atomicExch(status + ST_BAD_INDEX, 1); if (row_loss) row_loss[row] = 0.f; }
    return;
  }
  const bool vec = ((ld & 3) == 0) && ((classes & 3) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const Acc z_target = (Acc)z[target];  // read before pass 2 may overwrite an aliased row
  Acc mx = -INFINITY;
  if (vec) {
    for (int c = threadIdx.x * 4; c < classes; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(z + c);
      mx = max(mx, (Acc)max(max(v.x, v.y), max(v.z, v.w)));
    }
  } else {
    for (int c = threadIdx.x; c < classes; c += blockDim.x) mx = max(mx, (Acc)z[c]);
  }
  mx = block_max(mx, sm, (Acc)-INFINITY);
  Acc sum = 0;
  if (vec) {
    for (int c = threadIdx.x * 4; c < classes; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(z + c);
      sum += exp((Acc)v.x - mx) + exp((Acc)v.y - mx) + exp((Acc)v.z - mx) + exp((Acc)v.w - mx);
    }
  } else {
    for (int c = threadIdx.x; c < classes; c += blockDim.x) sum += exp((Acc)z[c] - mx);
  }
  sum = block_sum(sum, sm);
  if (threadIdx.x == 0 && row_loss) row_loss[row] = (float)(-z_target + mx + log(sum));
  if (dlogits == nullptr) return;
  const Acc inv = (Acc)1 / sum;
  const Acc sc = (Acc)scale;
  DT* d = dlogits + (size_t)row * ld_d;
  const bool vec_out = vec && ((ld_d & 3) == 0);
  if (vec_out) {
    for (int c = threadIdx.x * 4; c < classes; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(z + c);
      float o[4] = {(float)(exp((Acc)v.x - mx) * inv), (float)(exp((Acc)v.y - mx) * inv),
                    (float)(exp((Acc)v.z - mx) * inv), (float)(exp((Acc)v.w - mx) * inv)};
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = (float)(((Acc)o[e] - ((c + e) == target ? (Acc)1 : (Acc)0)) * sc);
      Vec<DT>::store(d + c, o);
    }
  } else {
    for (int c = threadIdx.x; c < classes; c += blockDim.x) {
      const Acc p = exp((Acc)z[c] - mx) * inv;
      store1(d + c, (float)((p - (c == target ? (Acc)1 : (Acc)0)) * sc));
    }
  }
}

// bf16-gradient route: persistent blocks walk rows, so only a few hundred rows (tens of MB)
// are in flight and the second read of a row is served by L2.  Pass 1 is an online
// max / sum-of-exponentials (one read), pass 2 writes dlogits = (softmax - onehot) * scale.
// Both passes are bound by load latency (DRAM in pass 1, L2 in pass 2), so each thread keeps U 16-byte loads in
// flight: at 50304 classes U = 7 takes the row in four rounds of even length and runs 10 % faster than U = 4
// (902 against 1007 us for 16384 rows); 8, 9 and 13 are slower again (ragged last round, registers).
constexpr int CE_THREADS = 512;
constexpr int CE_UNROLL = 7;
__global__ void __launch_bounds__(CE_THREADS, 2)
cross_entropy_online_kernel(const float* __restrict__ logits, long long ld, const int64_t* __restrict__ targets,
                            int rows, int classes, float scale, float* __restrict__ row_loss,
                            __nv_bfloat16* __restrict__ dlogits, long long ld_d, int* __restrict__ status) {
  __shared__ float sm[32];
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr int STEP = CE_THREADS * 4;  // columns covered by one 16-byte load per thread
  constexpr int U = CE_UNROLL;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* z = logits + (size_t)row * ld;
    const long long target = targets[row];
    if (target < 0 || target >= classes) {
      if (threadIdx.x == 0) { atomicExch(status + ST_BAD_INDEX, 1); if (row_loss) row_loss[row] = 0.f; }
      continue;
    }
    const float z_target = z[target];  // read before pass 2 may overwrite an aliased buffer
    // pass 1: U independent 16-byte loads per thread and step, one rescale of the running sum per step
    float m = -INFINITY, s = 0.f;  // m in units of log2(e) * logit
    for (int c0 = threadIdx.x * 4; c0 < classes; c0 += U * STEP) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u * STEP;
        v[u] = c < classes ? *reinterpret_cast<const float4*>(z + c) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
      float mx = -INFINITY;
#pragma unroll
      for (int u = 0; u < U; ++u) mx = fmaxf(mx, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
      mx *= kLog2e;
      if (mx > m) { s *= ex2_fast(m - mx); m = mx; }
#pragma unroll
      for (int u = 0; u < U; ++u)
        s += ex2_fast(fmaf(v[u].x, kLog2e, -m)) + ex2_fast(fmaf(v[u].y, kLog2e, -m)) + ex2_fast(fmaf(v[u].z, kLog2e, -m)) +
             ex2_fast(fmaf(v[u].w, kLog2e, -m));
    }
    const float big = block_max(m, sm, -INFINITY);
    const float total = block_sum(s * ex2_fast(m - big), sm);
    if (threadIdx.x == 0 && row_loss) row_loss[row] = -z_target + big * 0.6931471805599453f + logf(total);
    if (dlogits != nullptr) {
      const float inv = scale / total;
      __nv_bfloat16* d = dlogits + (size_t)row * ld_d;
      for (int c0 = threadIdx.x * 4; c0 < classes; c0 += U * STEP) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + u * STEP;
          v[u] = c < classes ? *reinterpret_cast<const float4*>(z + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + u * STEP;
          if (c < classes) {
            float o[4] = {ex2_fast(fmaf(v[u].x, kLog2e, -big)) * inv, ex2_fast(fmaf(v[u].y, kLog2e, -big)) * inv,
                          ex2_fast(fmaf(v[u].z, kLog2e, -big)) * inv, ex2_fast(fmaf(v[u].w, kLog2e, -big)) * inv};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (c + e == target) o[e] -= scale;
            Vec<__nv_bfloat16>::store(d + c, o);
          }
        }
      }
    }
    __syncthreads();  // sm is reused by the next row
  }
}

__global__ void mean_rows_kernel(const float* __restrict__ row_loss, int rows, float* __restrict__ out) {
  __shared__ double sm[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < rows; i += blockDim.x) acc += (double)row_loss[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) out[0] = (float)(acc / (double)rows);
}

}  // namespace

int layer_norm_forward_impl(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* beta, void* y,
                            int y_dtype, float* mean, float* rstd, int rows, int features, float eps) {
  HL_REQUIRE(ctx && x && gamma && beta && y, "hl_layer_norm_forward: null argument");
  HL_REQUIRE(rows > 0 && features > 0, "hl_layer_norm_forward: rows and features must be positive");
  HL_REQUIRE(eps > 0.f, "hl_layer_norm_forward: eps must be positive");
  ProfileScope prof(ctx, HL_PROF_LAYER_NORM, (double)rows * features * (double)(dtype_size(x_dtype) + dtype_size(y_dtype)));
  if (layer_norm_fast_applicable(x_dtype, y_dtype, features, x, y) &&
      ((reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15) == 0)
    return layer_norm_forward_fast(ctx, x, gamma, beta, y, mean, rstd, rows, features, eps);
  const int warps = 4;
  const int grid = ceil_div(rows, warps);
  const bool vec = (features % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(y) & 15) == 0) && ((reinterpret_cast<uintptr_t>(gamma) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(beta) & 15) == 0);
#define HL_LN_FWD(XT, YT, ACC)                                                                              \
  do {                                                                                                      \
    if (vec)                                                                                                \
      layer_norm_fwd_kernel<XT, YT, ACC, true><<<grid, warps * 32, 0, ctx->stream>>>(                       \
          (const XT*)x, gamma, beta, (YT*)y, mean, rstd, rows, features, eps);                              \
    else                                                                                                    \
      layer_norm_fwd_kernel<XT, YT, ACC, false><<<grid, warps * 32, 0, ctx->stream>>>(                      \
          (const XT*)x, gamma, beta, (YT*)y, mean, rstd, rows, features, eps);                              \
  } while (0)
  if (x_dtype == HL_F32 && y_dtype == HL_F32) HL_LN_FWD(float, float, double);
  else if (x_dtype == HL_BF16 && y_dtype == HL_BF16) HL_LN_FWD(__nv_bfloat16, __nv_bfloat16, float);
  else if (x_dtype == HL_F32 && y_dtype == HL_BF16) HL_LN_FWD(float, __nv_bfloat16, float);
  else if (x_dtype == HL_BF16 && y_dtype == HL_F32) HL_LN_FWD(__nv_bfloat16, float, float);
  else return fail("hl_layer_norm_forward: dtypes must be f32 or bf16");
#undef HL_LN_FWD
  HL_LAUNCH_CHECK("layer_norm_fwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int layer_norm_backward_impl(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* dy,
                             const float* mean, const float* rstd, const float* residual_grad, float* dx_f32,
                             void* dx_bf16, float* dgamma, float* dbeta, float* dx_colsum, int rows, int features,
                             FoldBatch* defer) {
  HL_REQUIRE(ctx && x && gamma && dy, "hl_layer_norm_backward: null argument");
  HL_REQUIRE(rows > 0 && features > 0, "hl_layer_norm_backward: rows and features must be positive");
  HL_REQUIRE(features % 4 == 0 && features <= LNB_MAXJ * 128,
             "hl_layer_norm_backward: features must be a multiple of 4 and at most 1024");
  HL_REQUIRE(x_dtype == HL_F32 || x_dtype == HL_BF16, "hl_layer_norm_backward: x dtype must be f32 or bf16");
  ProfileScope prof(ctx, HL_PROF_LAYER_NORM,
                    (double)rows * features * (double)(dtype_size(x_dtype) + 4 + (residual_grad ? 4 : 0) + (dx_f32 ? 4 : 0) + (dx_bf16 ? 2 : 0)));
  const uintptr_t align_bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gamma) |
                               reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(residual_grad) |
                               reinterpret_cast<uintptr_t>(dx_f32) | reinterpret_cast<uintptr_t>(dx_bf16);
  if (x_dtype == HL_BF16 && mean && rstd && features % 8 == 0 && (align_bits & 15) == 0)
    return layer_norm_backward_fast(ctx, x, gamma, dy, mean, rstd, residual_grad, dx_f32, dx_bf16, dgamma, dbeta,
                                    dx_colsum, rows, features, defer);
  HL_REQUIRE(!dx_colsum || dx_f32, "hl_layer_norm_backward: dx_colsum needs dx_f32 on this route");
  int blocks = std::min(ctx->sm_count * 2, ceil_div(rows, LNB_WARPS));
  const int rows_per_block = ceil_div(rows, blocks);
  blocks = ceil_div(rows, rows_per_block);
  int rc = ensure_workspace(ctx, sizeof(float) * (size_t)blocks * 2 * features);
  if (rc != HL_OK) return rc;
  float* partial = reinterpret_cast<float*>(ctx->workspace);
  const size_t smem = sizeof(float) * LNB_WARPS * 2 * (size_t)features;
  if (x_dtype == HL_F32) {
    auto k = layer_norm_bwd_kernel<float, double>;
    HL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<blocks, LNB_WARPS * 32, smem, ctx->stream>>>((const float*)x, gamma, dy, mean, rstd, residual_grad, dx_f32,
                                                      (__nv_bfloat16*)dx_bf16, partial, rows, features,
                                                      rows_per_block, 1e-5f);
  } else {
    auto k = layer_norm_bwd_kernel<__nv_bfloat16, float>;
    HL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<blocks, LNB_WARPS * 32, smem, ctx->stream>>>((const __nv_bfloat16*)x, gamma, dy, mean, rstd, residual_grad,
                                                      dx_f32, (__nv_bfloat16*)dx_bf16, partial, rows, features,
                                                      rows_per_block, 1e-5f);
  }
  HL_LAUNCH_CHECK("layer_norm_bwd_kernel");
  if (dgamma || dbeta) {
    layer_norm_bwd_fold_kernel<<<ceil_div(2 * features, 256), 256, 0, ctx->stream>>>(partial, dgamma, dbeta, features,
                                                                                      blocks);
    HL_LAUNCH_CHECK("layer_norm_bwd_fold_kernel");
    count_launch(ctx);
  }
  count_launch(ctx);
  if (dx_colsum) return bias_grad_impl(ctx, dx_f32, HL_F32, dx_colsum, rows, features);
  return HL_OK;
}

int cross_entropy_impl(hl_ctx* ctx, const float* logits, long long ld, const int64_t* targets, int rows, int classes,
                       float grad_scale, float* loss_dev, float* row_loss, void* dlogits, int dlogits_dtype,
                       long long ld_dlogits) {
  HL_REQUIRE(ctx && logits && targets, "hl_cross_entropy: null argument");
  HL_REQUIRE(rows > 0 && classes > 0, "hl_cross_entropy: requires non-empty batch/classes");
  HL_REQUIRE(ld >= classes, "hl_cross_entropy: row stride smaller than the class count");
  if (dlogits) {
    HL_REQUIRE(dlogits_dtype == HL_F32 || dlogits_dtype == HL_BF16, "hl_cross_entropy: dlogits dtype must be f32 or bf16");
    HL_REQUIRE(ld_dlogits >= classes, "hl_cross_entropy: dlogits row stride smaller than the class count");
  }
  float* rl = row_loss;
  if (!rl) {
    int rc = ensure_workspace(ctx, sizeof(float) * (size_t)rows);
    if (rc != HL_OK) return rc;
    rl = reinterpret_cast<float*>(ctx->workspace);
  }
  const float scale = grad_scale / (float)rows;
  ProfileScope prof(ctx, HL_PROF_LOSS, (double)rows * classes * (4.0 + (dlogits ? (double)dtype_size(dlogits_dtype) : 0.0)));
  const int threads = classes >= 4096 ? 512 : 256;
  const bool online_ok = (!dlogits || dlogits_dtype == HL_BF16) && classes % 4 == 0 && ld % 4 == 0 && ld_dlogits % 4 == 0 &&
                         (reinterpret_cast<uintptr_t>(logits) & 15) == 0 && (reinterpret_cast<uintptr_t>(dlogits) & 7) == 0 &&
                         classes >= 1024;
  if (online_ok && (dlogits || dlogits_dtype == HL_BF16))
    cross_entropy_online_kernel<<<std::min(rows, ctx->sm_count * 2), CE_THREADS, 0, ctx->stream>>>(
        logits, ld, targets, rows, classes, scale, rl, (__nv_bfloat16*)dlogits, ld_dlogits, ctx->status_dev);
  else if (dlogits && dlogits_dtype == HL_BF16)
    cross_entropy_kernel<float, __nv_bfloat16><<<rows, threads, 0, ctx->stream>>>(
        logits, ld, targets, rows, classes, scale, rl, (__nv_bfloat16*)dlogits, ld_dlogits, ctx->status_dev);
  else
    cross_entropy_kernel<double, float><<<rows, threads, 0, ctx->stream>>>(
        logits, ld, targets, rows, classes, scale, rl, (float*)dlogits, ld_dlogits, ctx->status_dev);
  HL_LAUNCH_CHECK("cross_entropy_kernel");
  count_launch(ctx);
  if (loss_dev) {
    mean_rows_kernel<<<1, 1024, 0, ctx->stream>>>(rl, rows, loss_dev);
    HL_LAUNCH_CHECK("mean_rows_kernel");
    count_launch(ctx);
  }
  return HL_OK;
}

}  // namespace hl

using namespace hl;

extern "C" {

int hl_layer_norm_forward(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* beta, void* y,
                          int y_dtype, float* mean, float* rstd, int rows, int features, float eps) {
  return layer_norm_forward_impl(ctx, x, x_dtype, gamma, beta, y, y_dtype, mean, rstd, rows, features, eps);
}

int hl_layer_norm_backward(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* dy,
                           const float* mean, const float* rstd, const float* residual_grad, float* dx_f32,
                           void* dx_bf16, float* dgamma, float* dbeta, float* dx_colsum, int rows, int features) {
  return layer_norm_backward_impl(ctx, x, x_dtype, gamma, dy, mean, rstd, residual_grad, dx_f32, dx_bf16, dgamma,
                                  dbeta, dx_colsum, rows, features);
}

int hl_embedding_forward(hl_ctx* ctx, const float* table, int table_rows, const int64_t* idx, const float* pos_table,
                         int period, void* out, int out_dtype, int n, int dim) {
  HL_REQUIRE(ctx && table && idx && out, "hl_embedding_forward: null argument");
  HL_REQUIRE(n > 0 && dim > 0 && table_rows > 0, "hl_embedding_forward: sizes must be positive");
  HL_REQUIRE(!pos_table || period > 0, "hl_embedding_forward: period must be positive with a position table");
  ProfileScope prof(ctx, HL_PROF_EMBEDDING, (double)n * dim * (4.0 + (pos_table ? 4.0 : 0.0) + (double)dtype_size(out_dtype)));
  const int warps = 4;
  if (out_dtype == HL_BF16)
    embedding_fwd_kernel<__nv_bfloat16><<<ceil_div(n, warps), warps * 32, 0, ctx->stream>>>(
        table, table_rows, idx, pos_table, period, (__nv_bfloat16*)out, n, dim, true, ctx->status_dev);
  else if (out_dtype == HL_F32)
    embedding_fwd_kernel<float><<<ceil_div(n, warps), warps * 32, 0, ctx->stream>>>(
        table, table_rows, idx, pos_table, period, (float*)out, n, dim, false, ctx->status_dev);
  else
    return fail("hl_embedding_forward: output dtype must be f32 or bf16");
  HL_LAUNCH_CHECK("embedding_fwd_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_embedding_backward(hl_ctx* ctx, const float* grad_out, const int64_t* idx, float* grad_table, int table_rows,
                          float* pos_grad, int period, int n, int dim) {
  HL_REQUIRE(ctx && grad_out && idx && grad_table, "hl_embedding_backward: null argument");
  HL_REQUIRE(n > 0 && dim > 0 && table_rows > 0, "hl_embedding_backward: sizes must be positive");
  ProfileScope prof(ctx, HL_PROF_EMBEDDING, (double)n * dim * 12.0);
  const int warps = 4;
  embedding_bwd_kernel<<<ceil_div(n, warps), warps * 32, 0, ctx->stream>>>(grad_out, idx, grad_table, table_rows, n,
                                                                           dim, ctx->status_dev);
  HL_LAUNCH_CHECK("embedding_bwd_kernel");
  count_launch(ctx);
  if (pos_grad) {
    HL_REQUIRE(period > 0, "hl_embedding_backward: period must be positive with a position gradient");
    const size_t total = (size_t)period * dim;
    position_grad_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(grad_out, pos_grad, period, n, dim);
    HL_LAUNCH_CHECK("position_grad_kernel");
    count_launch(ctx);
  }
  return HL_OK;
}

int hl_cross_entropy(hl_ctx* ctx, const float* logits, long long ld, const int64_t* targets, int rows, int classes,
                     float grad_scale, float* loss_dev, float* row_loss, void* dlogits, int dlogits_dtype,
                     long long ld_dlogits) {
  return cross_entropy_impl(ctx, logits, ld, targets, rows, classes, grad_scale, loss_dev, row_loss, dlogits,
                            dlogits_dtype, ld_dlogits);
}

}  // extern "C"
