// Bandwidth-bound row kernels of the bf16 route: layer norm forward/backward with the whole
// row held in registers (one global read per operand, 128-bit accesses) and a vectorised
// column-sum for bias gradients.  The backward also returns the column sums of the dx it
// writes, which is the bias gradient of the linear layer that produced that activation, so the
// f32 bias gradients of the step cost no extra pass over memory.
// Arithmetic: src/tensor.rs:3175-3256 (forward), src/tensor/autograd.rs:2158-2232 (backward),
// kernels.ptx:312 (bias gradient), in f32 as the reference's CUDA route.
#include "kernels.h"

namespace hl {
namespace {

constexpr int ROW_WARPS = 8;

__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y), c = unpack_bf16x2(t.z), d = unpack_bf16x2(t.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void load8_f32(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8_bf16(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) =
      make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}
__device__ __forceinline__ void store8_f32(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

__device__ __forceinline__ void unpack8_bf16(const uint4& t, float (&v)[8]) {
  const float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y), c = unpack_bf16x2(t.z), d = unpack_bf16x2(t.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}

// One warp per row, rows taken grid-stride; lane owns columns (j*32 + lane)*8 .. +7 for j < J.  The
// next row of the warp is requested before the current one is reduced.
template <int J>
__global__ void __launch_bounds__(ROW_WARPS * 32)
ln_fwd_bf16_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                   int features, float eps) {
  const int lane = threadIdx.x & 31;
  const int stride = gridDim.x * ROW_WARPS;
  int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  uint4 raw[J];
  auto fetch = [&](int r) {
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = (j * 32 + lane) * 8;
      raw[j] = (r < rows && c < features) ? *reinterpret_cast<const uint4*>(x + (size_t)r * features + c)
                                          : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch(row);
  for (; row < rows; row += stride) {
    float v[J][8];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      unpack8_bf16(raw[j], v[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += v[j][e];  // columns past the end hold zeros
    }
    fetch(row + stride);
    const float mean = warp_sum(sum) / (float)features;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < features) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float d = v[j][e] - mean; sq += d * d; }
      }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)features + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    __nv_bfloat16* yr = y + (size_t)row * features;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < features) {
        float g[8], b[8], o[8];
        load8_f32(gamma + c, g);
        load8_f32(beta + c, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (v[j][e] - mean) * rstd * g[e] + b[e];
        store8_bf16(yr + c, o);
      }
    }
  }
}

// Layer-norm backward.  A row is shared by WPR warps (a thread owns 8 consecutive columns, so its
// running column sums fit in 24 registers and many warps stay resident); a CTA holds several such
// row groups, each walking its share of the block's slab.  partial[block][3][features] receives the
// block's sums of dy*xhat, dy and of the dx written.
template <int WPR>
struct LnBwdShape {
  static constexpr int GROUPS = (WPR >= 3) ? 12 / WPR : 8 / WPR;
  static constexpr int THREADS = GROUPS * WPR * 32;
  static_assert(WPR == 1 || GROUPS <= 4, "one hardware barrier per row group");
};

template <int WPR>
__global__ void __launch_bounds__(LnBwdShape<WPR>::THREADS, 2)
ln_bwd_bf16_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ dy,
                   const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                   const float* __restrict__ residual, float* __restrict__ dx_f32, __nv_bfloat16* __restrict__ dx_bf16,
                   float* __restrict__ partial, int rows, int features, int rows_per_block) {
  constexpr int GROUPS = LnBwdShape<WPR>::GROUPS;
  extern __shared__ float fold_smem[];  // [GROUPS][3][features]
  __shared__ float2 row_sums[2][GROUPS][WPR];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp / WPR, wr = warp % WPR;
  const int c = (wr * 32 + lane) * 8;
  const bool active = c < features;
  const int r0 = blockIdx.x * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float g[8], dg[8], db[8], ds[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { g[e] = 0.f; dg[e] = 0.f; db[e] = 0.f; ds[e] = 0.f; }
  if (active) load8_f32(gamma + c, g);
  const float inv_f = 1.0f / (float)features;
  int parity = 0;
  for (int row = r0 + group; row < r1; row += GROUPS, parity ^= 1) {
    const size_t base = (size_t)row * features + c;
    float xh[8], d[8], o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { xh[e] = 0.f; d[e] = 0.f; o[e] = 0.f; }
    if (active) {  // every global read of the row is issued before anything is consumed
      load8_bf16(x + base, xh);
      load8_f32(dy + base, d);
      if (residual) load8_f32(residual + base, o);
    }
    const float mean = mean_in[row], rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
    if (active) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xh[e] = (xh[e] - mean) * rstd;
        dg[e] += d[e] * xh[e];
        db[e] += d[e];
        d[e] *= g[e];  // dxhat
        s1 += d[e];
        s2 += d[e] * xh[e];
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if constexpr (WPR > 1) {
      if (lane == 0) row_sums[parity][group][wr] = make_float2(s1, s2);
      // hardware barrier 1 + group, immediate ids so that a CTA reserves only GROUPS + 1 of the SM's 16
      switch (group) {
        case 0: asm volatile("bar.sync 1, %0;" ::"n"(WPR * 32) : "memory"); break;
        case 1: asm volatile("bar.sync 2, %0;" ::"n"(WPR * 32) : "memory"); break;
        case 2: asm volatile("bar.sync 3, %0;" ::"n"(WPR * 32) : "memory"); break;
        default: asm volatile("bar.sync 4, %0;" ::"n"(WPR * 32) : "memory"); break;
      }
      s1 = 0.f;
      s2 = 0.f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) {
        const float2 t = row_sums[parity][group][w];
        s1 += t.x;
        s2 += t.y;
      }
    }
    if (active) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float dxv = rstd * ((float)features * d[e] - s1 - xh[e] * s2) * inv_f;
        o[e] = residual ? o[e] + dxv : dxv;
        ds[e] += o[e];
      }
      if (dx_f32) store8_f32(dx_f32 + base, o);
      if (dx_bf16) store8_bf16(dx_bf16 + base, o);
    }
  }
  if (active) {
    float* mine = fold_smem + (size_t)group * 3 * features + c;
    store8_f32(mine, dg);
    store8_f32(mine + features, db);
    store8_f32(mine + 2 * features, ds);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 3 * features; i += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < GROUPS; ++w) t += fold_smem[(size_t)w * 3 * features + i];
    partial[(size_t)blockIdx.x * 3 * features + i] = t;
  }
}

// Sum `blocks` partial rows of `total` columns each, in a fixed order (so the result does not depend
// on scheduling): a CTA owns 32 columns, its 32 warps take interleaved partial rows (all of a warp's
// loads are in flight together) and meet in shared memory.  Column c goes to o0/o1/o2 by
// c / features (null pointers are skipped).
constexpr int FOLD_WARPS = 32;
__global__ void __launch_bounds__(FOLD_WARPS * 32)
fold_partials_kernel(const float* __restrict__ partial, int blocks, int total, float* __restrict__ o0,
                     float* __restrict__ o1, float* __restrict__ o2, int features) {
  __shared__ double acc[FOLD_WARPS][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  double s = 0.0;
  if (c < total) {
    for (int b0 = warp; b0 < blocks; b0 += FOLD_WARPS * 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int b = b0 + u * FOLD_WARPS;
        v[u] = b < blocks ? partial[(size_t)b * total + c] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) s += (double)v[u];
    }
  }
  acc[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < total) {
#pragma unroll 8
    for (int w = 1; w < FOLD_WARPS; ++w) s += acc[w][lane];
    float* dst = c < features ? o0 : (c < 2 * features ? o1 : o2);
    if (dst) dst[c % features] = (float)s;
  }
}

// The same fold for up to FoldBatch::kMaxJobs reductions in one launch: blockIdx.y picks the job.
struct FoldJobs {
  FoldJob job[FoldBatch::kMaxJobs];
};
__global__ void __launch_bounds__(FOLD_WARPS * 32)
fold_batch_kernel(const FoldJobs jobs) {
  __shared__ double acc[FOLD_WARPS][33];
  const FoldJob& j = jobs.job[blockIdx.y];
  if ((int)blockIdx.x * 32 >= j.total) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  double s = 0.0;
  if (c < j.total) {
    for (int b0 = warp; b0 < j.blocks; b0 += FOLD_WARPS * 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int b = b0 + u * FOLD_WARPS;
        v[u] = b < j.blocks ? j.partial[(size_t)b * j.total + c] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) s += (double)v[u];
    }
  }
  acc[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < j.total) {
#pragma unroll 8
    for (int w = 1; w < FOLD_WARPS; ++w) s += acc[w][lane];
    float* dst = c < j.features ? j.o0 : (c < 2 * j.features ? j.o1 : j.o2);
    if (dst) dst[c % j.features] = (float)s;
  }
}

// Column sums with 16-byte loads: a warp covers 32*VEC consecutive columns, the block's eight
// warps take different rows of the slab.
template <typename T, int VEC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
colsum_vec_kernel(const T* __restrict__ g, float* __restrict__ partial, int rows, int cols, int rows_per_block) {
  __shared__ float fold[ROW_WARPS][32 * VEC + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * VEC;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
  if (c < cols) {
#pragma unroll 4
    for (int r = r0 + warp; r < r1; r += ROW_WARPS) {
      float v[8];
      if constexpr (VEC == 8) load8_bf16(reinterpret_cast<const __nv_bfloat16*>(g) + (size_t)r * cols + c, v);
      else {
        const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + (size_t)r * cols + c);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] += v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) fold[warp][lane * VEC + e] = acc[e];
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * VEC; i += blockDim.x) {
    const int col = blockIdx.x * 32 * VEC + i;
    if (col < cols) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < ROW_WARPS; ++w) s += fold[w][i];
      partial[(size_t)blockIdx.y * cols + col] = s;
    }
  }
}

}  // namespace

float* fold_batch_reserve(FoldBatch* batch, size_t elems) {
  if (!batch || !batch->scratch || batch->n >= FoldBatch::kMaxJobs) return nullptr;
  const size_t need = (elems + 63) & ~size_t(63);
  if (batch->used + need > batch->capacity) return nullptr;
  float* p = batch->scratch + batch->used;
  batch->used += need;
  return p;
}

void fold_batch_add(FoldBatch* batch, const float* partial, int blocks, int total, int features, float* o0, float* o1,
                    float* o2) {
  batch->jobs[batch->n++] = FoldJob{partial, blocks, total, features, o0, o1, o2};
}

int fold_batch_flush(hl_ctx* ctx, FoldBatch* batch) {
  if (!batch || batch->n == 0) return HL_OK;
  FoldJobs jobs{};
  int widest = 0;
  for (int i = 0; i < batch->n; ++i) {
    jobs.job[i] = batch->jobs[i];
    widest = std::max(widest, batch->jobs[i].total);
  }
  fold_batch_kernel<<<dim3(ceil_div(widest, 32), batch->n), FOLD_WARPS * 32, 0, ctx->stream>>>(jobs);
  HL_LAUNCH_CHECK("fold_batch_kernel");
  count_launch(ctx);
  batch->n = 0;
  batch->used = 0;
  return HL_OK;
}

bool layer_norm_fast_applicable(int x_dtype, int y_dtype, int features, const void* x, const void* y) {
  return x_dtype == HL_BF16 && y_dtype == HL_BF16 && features % 8 == 0 && features <= 1024 &&
         ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
}

int layer_norm_forward_fast(hl_ctx* ctx, const void* x, const float* gamma, const float* beta, void* y, float* mean,
                            float* rstd, int rows, int features, float eps) {
  const int grid = std::min(ceil_div(rows, ROW_WARPS), ctx->sm_count * 8);
  const int J = ceil_div(features, 256);
#define HL_LAUNCH(JJ)                                                                                          \
  ln_fwd_bf16_kernel<JJ><<<grid, ROW_WARPS * 32, 0, ctx->stream>>>((const __nv_bfloat16*)x, gamma, beta,       \
                                                                    (__nv_bfloat16*)y, mean, rstd, rows, features, eps)
  switch (J) {
    case 1: HL_LAUNCH(1); break;
    case 2: HL_LAUNCH(2); break;
    case 3: HL_LAUNCH(3); break;
    default: HL_LAUNCH(4); break;
  }
#undef HL_LAUNCH
  HL_LAUNCH_CHECK("ln_fwd_bf16_kernel");
  count_launch(ctx);
  return HL_OK;
}

int layer_norm_backward_fast(hl_ctx* ctx, const void* x, const float* gamma, const float* dy, const float* mean,
                             const float* rstd, const float* residual, float* dx_f32, void* dx_bf16, float* dgamma,
                             float* dbeta, float* dx_colsum, int rows, int features, FoldBatch* defer) {
  const int wpr = ceil_div(features, 256);  // 1..4: a warp covers 256 columns
  const int groups = wpr >= 3 ? 12 / wpr : 8 / wpr;
  int blocks = std::min(2 * ctx->sm_count, ceil_div(rows, groups));
  const int rows_per_block = ceil_div(rows, blocks);
  blocks = ceil_div(rows, rows_per_block);
  float* partial = fold_batch_reserve(defer, (size_t)blocks * 3 * features);
  const bool deferred = partial != nullptr;
  if (!deferred) {
    int rc = ensure_workspace(ctx, sizeof(float) * (size_t)blocks * 3 * features);
    if (rc != HL_OK) return rc;
    partial = reinterpret_cast<float*>(ctx->workspace);
  }
  const size_t smem = sizeof(float) * (size_t)groups * 3 * features;  // at most 36 KB
#define HL_LAUNCH(W)                                                                                              \
  ln_bwd_bf16_kernel<W><<<blocks, LnBwdShape<W>::THREADS, smem, ctx->stream>>>(                                   \
      (const __nv_bfloat16*)x, gamma, dy, mean, rstd, residual, dx_f32, (__nv_bfloat16*)dx_bf16, partial, rows,   \
      features, rows_per_block)
  switch (wpr) {
    case 1: HL_LAUNCH(1); break;
    case 2: HL_LAUNCH(2); break;
    case 3: HL_LAUNCH(3); break;
    default: HL_LAUNCH(4); break;
  }
#undef HL_LAUNCH
  HL_LAUNCH_CHECK("ln_bwd_bf16_kernel");
  if (deferred) {
    fold_batch_add(defer, partial, blocks, 3 * features, features, dgamma, dbeta, dx_colsum);
    count_launch(ctx);
    return HL_OK;
  }
  fold_partials_kernel<<<ceil_div(3 * features, 32), FOLD_WARPS * 32, 0, ctx->stream>>>(partial, blocks, 3 * features, dgamma,
                                                                                     dbeta, dx_colsum, features);
  HL_LAUNCH_CHECK("fold_partials_kernel");
  count_launch(ctx, 2);
  return HL_OK;
}

bool colsum_fast_applicable(int dtype, int cols, const void* g) {
  const int vec = dtype == HL_BF16 ? 8 : 4;
  return (dtype == HL_BF16 || dtype == HL_F32) && cols % vec == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0;
}

int colsum_fast(hl_ctx* ctx, const void* g, int dtype, float* out, int rows, int cols, FoldBatch* defer) {
  const int vec = dtype == HL_BF16 ? 8 : 4;
  const int col_blocks = ceil_div(cols, 32 * vec);
  int slabs = std::max(1, std::min(std::min(64, ceil_div(rows, ROW_WARPS * 4)), (ctx->sm_count * 4) / col_blocks));
  const int rows_per_block = ceil_div(rows, slabs);
  slabs = ceil_div(rows, rows_per_block);
  float* partial = fold_batch_reserve(defer, (size_t)slabs * cols);
  const bool deferred = partial != nullptr;
  if (!deferred) {
    int rc = ensure_workspace(ctx, sizeof(float) * (size_t)slabs * cols);
    if (rc != HL_OK) return rc;
    partial = reinterpret_cast<float*>(ctx->workspace);
  }
  dim3 grid(col_blocks, slabs);
  if (dtype == HL_BF16)
    colsum_vec_kernel<__nv_bfloat16, 8><<<grid, ROW_WARPS * 32, 0, ctx->stream>>>((const __nv_bfloat16*)g, partial, rows,
                                                                                   cols, rows_per_block);
  else
    colsum_vec_kernel<float, 4><<<grid, ROW_WARPS * 32, 0, ctx->stream>>>((const float*)g, partial, rows, cols,
                                                                           rows_per_block);
  HL_LAUNCH_CHECK("colsum_vec_kernel");
  if (deferred) {
    fold_batch_add(defer, partial, slabs, cols, cols, out, nullptr, nullptr);
    count_launch(ctx);
    return HL_OK;
  }
  fold_partials_kernel<<<ceil_div(cols, 32), FOLD_WARPS * 32, 0, ctx->stream>>>(partial, slabs, cols, out, nullptr, nullptr,
                                                                             cols);
  HL_LAUNCH_CHECK("fold_partials_kernel");
  count_launch(ctx, 2);
  return HL_OK;
}

}  // namespace hl
