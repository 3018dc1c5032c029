// 128-bit vectorised elementwise kernels, casts, bias add / bias gradient and grid reductions.
// Reference counterparts are one-thread-per-element scalar PTX entries
// (heirloom-kernels/src/ptx/kernels.ptx:6-312, :4610-4907).
#include "kernels.h"

namespace hl {
namespace {

constexpr int EW_THREADS = 256;

inline int ew_grid(hl_ctx* ctx, size_t vec_items) {
  size_t blocks = (vec_items + EW_THREADS - 1) / EW_THREADS;
  size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

struct OpAdd { __device__ float operator()(float a, float b) const { return a + b; } };
struct OpSub { __device__ float operator()(float a, float b) const { return a - b; } };
struct OpMul { __device__ float operator()(float a, float b) const { return a * b; } };
struct OpDiv { __device__ float operator()(float a, float b) const { return a / b; } };

template <typename Op>
__global__ void binary_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                  size_t n, bool vec) {
  Op op;
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  if (vec) {
    const size_t n4 = n / 4;
    for (size_t i = tid; i < n4; i += stride) {
      const float4 x = reinterpret_cast<const float4*>(a)[i], y = reinterpret_cast<const float4*>(b)[i];
      reinterpret_cast<float4*>(out)[i] = make_float4(op(x.x, y.x), op(x.y, y.y), op(x.z, y.z), op(x.w, y.w));
    }
    for (size_t i = n4 * 4 + tid; i < n; i += stride) out[i] = op(a[i], b[i]);
  } else {
    for (size_t i = tid; i < n; i += stride) out[i] = op(a[i], b[i]);
  }
}

// Unary f32 map with an optional second input; F(x, y).
template <typename F>
__global__ void map_f32_kernel(const float* __restrict__ x, const float* __restrict__ y, float* __restrict__ out,
                               size_t n, bool vec, F f) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  if (vec) {
    const size_t n4 = n / 4;
    for (size_t i = tid; i < n4; i += stride) {
      const float4 a = x ? reinterpret_cast<const float4*>(x)[i] : make_float4(0, 0, 0, 0);
      const float4 b = y ? reinterpret_cast<const float4*>(y)[i] : make_float4(0, 0, 0, 0);
      reinterpret_cast<float4*>(out)[i] = make_float4(f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w));
    }
    for (size_t i = n4 * 4 + tid; i < n; i += stride) out[i] = f(x ? x[i] : 0.f, y ? y[i] : 0.f);
  } else {
    for (size_t i = tid; i < n; i += stride) out[i] = f(x ? x[i] : 0.f, y ? y[i] : 0.f);
  }
}

// bf16 map over 8-element vectors; F(x, y) in f32, result rounded to bf16.
template <typename F>
__global__ void map_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                __nv_bfloat16* __restrict__ out, size_t n, bool vec, F f) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  if (vec) {
    const size_t n8 = n / 8;
    for (size_t i = tid; i < n8; i += stride) {
      const uint4 a = reinterpret_cast<const uint4*>(x)[i];
      const uint4 b = y ? reinterpret_cast<const uint4*>(y)[i] : make_uint4(0, 0, 0, 0);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
      uint32_t ow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 af = unpack_bf16x2(aw[j]), bf = unpack_bf16x2(bw[j]);
        ow[j] = pack_bf16x2(f(af.x, bf.x), f(af.y, bf.y));
      }
      reinterpret_cast<uint4*>(out)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    for (size_t i = n8 * 8 + tid; i < n; i += stride)
      out[i] = to_bf16(f(from_bf16(x[i]), y ? from_bf16(y[i]) : 0.f));
  } else {
    for (size_t i = tid; i < n; i += stride) out[i] = to_bf16(f(from_bf16(x[i]), y ? from_bf16(y[i]) : 0.f));
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n,
                                        bool vec) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  if (vec) {
    const size_t n8 = n / 8;
    for (size_t i = tid; i < n8; i += stride) {
      const float4 a = reinterpret_cast<const float4*>(src)[2 * i], b = reinterpret_cast<const float4*>(src)[2 * i + 1];
      reinterpret_cast<uint4*>(dst)[i] =
          make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
    }
    for (size_t i = n8 * 8 + tid; i < n; i += stride) dst[i] = to_bf16(src[i]);
  } else {
    for (size_t i = tid; i < n; i += stride) dst[i] = to_bf16(src[i]);
  }
}

__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, size_t n,
                                        bool vec) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  if (vec) {
    const size_t n8 = n / 8;
    for (size_t i = tid; i < n8; i += stride) {
      const uint4 a = reinterpret_cast<const uint4*>(src)[i];
      const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      reinterpret_cast<float4*>(dst)[2 * i] = make_float4(f0.x, f0.y, f1.x, f1.y);
      reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(f2.x, f2.y, f3.x, f3.y);
    }
    for (size_t i = n8 * 8 + tid; i < n; i += stride) dst[i] = from_bf16(src[i]);
  } else {
    for (size_t i = tid; i < n; i += stride) dst[i] = from_bf16(src[i]);
  }
}

__global__ void bias_add_f32_kernel(const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ out,
                                    size_t total, int cols) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = tid; i < total; i += stride) out[i] = x[i] + bias[i % cols];
}

// Column sums, stage 1: each block owns a slab of rows and 32 columns; threads (32 x 8) walk
// rows with coalesced 32-wide reads, partial sums in double, then a shared-memory reduce.
template <typename T>
__global__ void colsum_partial_kernel(const T* __restrict__ g, double* __restrict__ partial, int rows, int cols,
                                      int rows_per_block) {
  __shared__ double tile[8][33];
  const int col = blockIdx.x * 32 + threadIdx.x;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  double acc = 0.0;
  if (col < cols) {
    for (int r = r0 + threadIdx.y; r < r1; r += 8) {
      float v;
      if constexpr (sizeof(T) == 2) v = from_bf16(g[(size_t)r * cols + col]);
      else v = g[(size_t)r * cols + col];
      acc += (double)v;
    }
  }
  tile[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < cols) {
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += tile[j][threadIdx.x];
    partial[(size_t)blockIdx.y * cols + col] = s;
  }
}

__global__ void colsum_final_kernel(const double* __restrict__ partial, float* __restrict__ out, int cols, int slabs) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  double s = 0.0;
  for (int j = 0; j < slabs; ++j) s += partial[(size_t)j * cols + col];
  out[col] = (float)s;
}

// Grid reduction: per-block double partial sums, last block (ticket) folds them in a fixed order.
template <int MODE>  // 0 sum, 1 sum of squares
__global__ void reduce_partial_kernel(const float* __restrict__ x, size_t n, double* __restrict__ partial) {
  __shared__ double sm[32];
  double acc = 0.0;
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = tid; i < n; i += stride) {
    const double v = (double)x[i];
    acc += MODE == 1 ? v * v : v;
  }
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

__global__ void reduce_final_kernel(const double* __restrict__ partial, int count, double scale, float* __restrict__ out) {
  __shared__ double sm[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < count; i += blockDim.x) acc += partial[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) out[0] = (float)(acc * scale);
}

int reduce_impl(hl_ctx* ctx, const float* x, size_t n, float* out_dev, int mode, double scale) {
  HL_REQUIRE(ctx && out_dev && (x || n == 0), "reduction: null argument");
  const int blocks = (int)std::min<size_t>(std::max<size_t>((n + 1023) / 1024, 1), (size_t)ctx->sm_count * 4);
  int rc = ensure_workspace(ctx, sizeof(double) * blocks);
  if (rc != HL_OK) return rc;
  double* partial = reinterpret_cast<double*>(ctx->workspace);
  if (mode == 1) reduce_partial_kernel<1><<<blocks, 256, 0, ctx->stream>>>(x, n, partial);
  else reduce_partial_kernel<0><<<blocks, 256, 0, ctx->stream>>>(x, n, partial);
  HL_LAUNCH_CHECK("reduce_partial_kernel");
  reduce_final_kernel<<<1, 256, 0, ctx->stream>>>(partial, blocks, scale, out_dev);
  HL_LAUNCH_CHECK("reduce_final_kernel");
  count_launch(ctx, 2);
  return HL_OK;
}

}  // namespace

int bias_grad_impl(hl_ctx* ctx, const void* grad_out, int dtype, float* grad_bias, int rows, int cols, FoldBatch* defer) {
  HL_REQUIRE(ctx && grad_out && grad_bias, "hl_bias_grad: null argument");
  HL_REQUIRE(rows > 0 && cols > 0, "hl_bias_grad: rows and cols must be positive");
  HL_REQUIRE(dtype == HL_F32 || dtype == HL_BF16, "hl_bias_grad: dtype must be f32 or bf16");
  ProfileScope prof(ctx, HL_PROF_BIAS_GRAD, (double)rows * cols * (double)dtype_size(dtype));
  if (colsum_fast_applicable(dtype, cols, grad_out)) return colsum_fast(ctx, grad_out, dtype, grad_bias, rows, cols, defer);
  int slabs = std::min(std::max(rows / 256, 1), 64);
  const int rows_per_block = ceil_div(rows, slabs);
  slabs = ceil_div(rows, rows_per_block);
  int rc = ensure_workspace(ctx, sizeof(double) * (size_t)slabs * cols);
  if (rc != HL_OK) return rc;
  double* partial = reinterpret_cast<double*>(ctx->workspace);
  dim3 grid(ceil_div(cols, 32), slabs), block(32, 8);
  if (dtype == HL_BF16)
    colsum_partial_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(grad_out), partial, rows, cols, rows_per_block);
  else
    colsum_partial_kernel<float><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const float*>(grad_out), partial,
                                                                    rows, cols, rows_per_block);
  HL_LAUNCH_CHECK("colsum_partial_kernel");
  colsum_final_kernel<<<ceil_div(cols, 256), 256, 0, ctx->stream>>>(partial, grad_bias, cols, slabs);
  HL_LAUNCH_CHECK("colsum_final_kernel");
  count_launch(ctx, 2);
  return HL_OK;
}

}  // namespace hl

using namespace hl;

extern "C" {

int hl_binary_f32(hl_ctx* ctx, int op, const float* a, const float* b, float* out, size_t n) {
  HL_REQUIRE(ctx && ((a && b && out) || n == 0), "hl_binary_f32: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(a) && aligned16(b) && aligned16(out);
  const int grid = ew_grid(ctx, vec ? n / 4 + 1 : n);
  switch (op) {
    case HL_ADD: binary_f32_kernel<OpAdd><<<grid, EW_THREADS, 0, ctx->stream>>>(a, b, out, n, vec); break;
    case HL_SUB: binary_f32_kernel<OpSub><<<grid, EW_THREADS, 0, ctx->stream>>>(a, b, out, n, vec); break;
    case HL_MUL: binary_f32_kernel<OpMul><<<grid, EW_THREADS, 0, ctx->stream>>>(a, b, out, n, vec); break;
    case HL_DIV: binary_f32_kernel<OpDiv><<<grid, EW_THREADS, 0, ctx->stream>>>(a, b, out, n, vec); break;
    default: return fail("hl_binary_f32: unknown op");
  }
  HL_LAUNCH_CHECK("binary_f32_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_scale_f32(hl_ctx* ctx, const float* a, float s, float* out, size_t n) {
  HL_REQUIRE(ctx && ((a && out) || n == 0), "hl_scale_f32: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(a) && aligned16(out);
  map_f32_kernel<<<ew_grid(ctx, vec ? n / 4 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
      a, (const float*)nullptr, out, n, vec, [s] __device__(float x, float) { return x * s; });
  HL_LAUNCH_CHECK("scale_f32");
  count_launch(ctx);
  return HL_OK;
}

int hl_fill_f32(hl_ctx* ctx, float* out, float value, size_t n) {
  HL_REQUIRE(ctx && (out || n == 0), "hl_fill_f32: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(out);
  map_f32_kernel<<<ew_grid(ctx, vec ? n / 4 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
      (const float*)nullptr, (const float*)nullptr, out, n, vec, [value] __device__(float, float) { return value; });
  HL_LAUNCH_CHECK("fill_f32");
  count_launch(ctx);
  return HL_OK;
}

// ---- plain SGD, index ranges and index concatenation ---------------------------------------------------------
static __global__ void sgd_update_kernel(float* __restrict__ param, const float* __restrict__ grad, float lr, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    param[i] = __fsub_rn(param[i], __fmul_rn(lr, grad[i]));  // two roundings, as the reference's mul then sub
}
static __global__ void arange_i64_kernel(int64_t* __restrict__ out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = (int64_t)i;
}
static __global__ void copy_i64_kernel(const int64_t* __restrict__ src, int64_t* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

int hl_sgd_update_f32(hl_ctx* ctx, float* param, const float* grad, float lr, size_t n) {
  HL_REQUIRE(ctx && ((param && grad) || n == 0), "hl_sgd_update_f32: null argument");
  HL_REQUIRE(lr > 0.f, "sgd_update_f32_buffer learning rate must be positive, got " + std::to_string(lr));
  if (n == 0) return HL_OK;
  sgd_update_kernel<<<ew_grid(ctx, n), EW_THREADS, 0, ctx->stream>>>(param, grad, lr, n);
  HL_LAUNCH_CHECK("sgd_update_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_arange_i64(hl_ctx* ctx, int64_t* out, size_t n) {
  HL_REQUIRE(ctx && (out || n == 0), "hl_arange_i64: null argument");
  HL_REQUIRE(n <= 0xffffffffull, "i64_arange len exceeds the u32 launch limit");
  if (n == 0) return HL_OK;
  arange_i64_kernel<<<ew_grid(ctx, n), EW_THREADS, 0, ctx->stream>>>(out, n);
  HL_LAUNCH_CHECK("arange_i64_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_concat_i64(hl_ctx* ctx, const int64_t* const* inputs, const size_t* lengths, int count, int64_t* out, size_t out_capacity) {
  HL_REQUIRE(ctx && inputs && lengths, "hl_concat_i64: null argument");
  HL_REQUIRE(count >= 1, "concat_i64_buffers requires at least one input buffer");
  size_t total = 0;
  for (int i = 0; i < count; ++i) {
    HL_REQUIRE(lengths[i] == 0 || inputs[i], "hl_concat_i64: null input buffer");
    HL_REQUIRE(total + lengths[i] >= total, "concat_i64_buffers total length overflow");
    total += lengths[i];
  }
  HL_REQUIRE(total <= out_capacity, "hl_concat_i64: the output holds " + std::to_string(out_capacity) + " elements, the inputs " +
                                        std::to_string(total));
  HL_REQUIRE(out || total == 0, "hl_concat_i64: null output");
  size_t offset = 0;
  for (int i = 0; i < count; ++i) {
    if (lengths[i] == 0) continue;
    copy_i64_kernel<<<ew_grid(ctx, lengths[i]), EW_THREADS, 0, ctx->stream>>>(inputs[i], out + offset, lengths[i]);
    HL_LAUNCH_CHECK("copy_i64_kernel");
    count_launch(ctx);
    offset += lengths[i];
  }
  return HL_OK;
}

int hl_relu_f32(hl_ctx* ctx, const float* x, float* out, size_t n) {
  HL_REQUIRE(ctx && ((x && out) || n == 0), "hl_relu_f32: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(x) && aligned16(out);
  map_f32_kernel<<<ew_grid(ctx, vec ? n / 4 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
      x, (const float*)nullptr, out, n, vec, [] __device__(float v, float) { return v > 0.f ? v : 0.f; });
  HL_LAUNCH_CHECK("relu_f32");
  count_launch(ctx);
  return HL_OK;
}

int hl_relu_backward_f32(hl_ctx* ctx, const float* x, const float* grad_out, float* grad_in, size_t n) {
  HL_REQUIRE(ctx && ((x && grad_out && grad_in) || n == 0), "hl_relu_backward_f32: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(x) && aligned16(grad_out) && aligned16(grad_in);
  map_f32_kernel<<<ew_grid(ctx, vec ? n / 4 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
      x, grad_out, grad_in, n, vec, [] __device__(float v, float g) { return v > 0.f ? g : 0.f; });
  HL_LAUNCH_CHECK("relu_backward_f32");
  count_launch(ctx);
  return HL_OK;
}

int hl_cast(hl_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, size_t n) {
  HL_REQUIRE(ctx && ((src && dst) || n == 0), "hl_cast: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(src) && aligned16(dst);
  const int grid = ew_grid(ctx, vec ? n / 8 + 1 : n);
  if (src_dtype == HL_F32 && dst_dtype == HL_BF16) {
    cast_f32_to_bf16_kernel<<<grid, EW_THREADS, 0, ctx->stream>>>((const float*)src, (__nv_bfloat16*)dst, n, vec);
  } else if (src_dtype == HL_BF16 && dst_dtype == HL_F32) {
    cast_bf16_to_f32_kernel<<<grid, EW_THREADS, 0, ctx->stream>>>((const __nv_bfloat16*)src, (float*)dst, n, vec);
  } else if (src_dtype == HL_F32 && dst_dtype == HL_F32) {
    map_f32_kernel<<<ew_grid(ctx, vec ? n / 4 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
        (const float*)src, (const float*)nullptr, (float*)dst, n, vec,
        [] __device__(float v, float) { return bf16_round(v); });
  } else {
    return fail("hl_cast: supported pairs are f32->bf16, bf16->f32 and the f32 bf16-round-trip");
  }
  HL_LAUNCH_CHECK("cast kernel");
  count_launch(ctx);
  return HL_OK;
}

// One f32 value as a sum of bf16 pieces: hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid).  The
// differences are exact in f32, so hi + mid + lo == x whenever the three 8-bit mantissas reach the last bit of x.
static __global__ void split_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows, int cols,
                                  int mode_bits) {
  const int mode = mode_bits & 3;
  const bool stacked = (mode_bits & HL_SPLIT_STACK_ROWS) != 0;
  const int pieces = mode == HL_SPLIT_HI_LO ? 2 : 3;
  const long long n = rows * cols;
  const long long piece_stride = stacked ? n : cols;            // distance between the pieces of one element
  const long long ld = stacked ? cols : (long long)pieces * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = (int)(i - r * cols);
    const float x = src[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    __nv_bfloat16* out = dst + r * ld + c;
    out[0] = hi;
    if (mode == HL_SPLIT_HI_MID_LO) { out[piece_stride] = mid; out[2 * piece_stride] = lo; }
    else if (mode == HL_SPLIT_HI_HI_LO) { out[piece_stride] = hi; out[2 * piece_stride] = mid; }
    else out[piece_stride] = mid;
  }
}

int hl_split_bf16_f32(hl_ctx* ctx, const float* src, void* dst, long long rows, int cols, int mode) {
  HL_REQUIRE(ctx && src && dst, "hl_split_bf16_f32: null argument");
  HL_REQUIRE(rows > 0 && cols > 0, "hl_split_bf16_f32: requires non-zero rows/cols");
  HL_REQUIRE((mode & ~(3 | HL_SPLIT_STACK_ROWS)) == 0 && (mode & 3) != 3, "hl_split_bf16_f32: unknown mode");
  split_bf16_kernel<<<ew_grid(ctx, (size_t)rows * cols), EW_THREADS, 0, ctx->stream>>>(src, (__nv_bfloat16*)dst, rows, cols, mode);
  HL_LAUNCH_CHECK("split_bf16_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_gelu(hl_ctx* ctx, const void* x, void* out, int dtype, size_t n) {
  HL_REQUIRE(ctx && ((x && out) || n == 0), "hl_gelu: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(x) && aligned16(out);
  if (dtype == HL_F32) {
    // f32 tensors are evaluated in double so the f32 result is correctly rounded from the
    // same f64 expression the reference evaluates.
    map_f32_kernel<<<ew_grid(ctx, vec ? n / 4 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
        (const float*)x, (const float*)nullptr, (float*)out, n, vec,
        [] __device__(float v, float) { return (float)gelu_fwd<double>((double)v); });
  } else if (dtype == HL_BF16) {
    map_bf16_kernel<<<ew_grid(ctx, vec ? n / 8 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)out, n, vec,
        [] __device__(float v, float) { return gelu_fwd_f(v); });
  } else {
    return fail("hl_gelu: dtype must be f32 or bf16");
  }
  HL_LAUNCH_CHECK("gelu kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_gelu_backward(hl_ctx* ctx, const void* x, const void* grad_out, void* grad_in, int dtype, size_t n) {
  HL_REQUIRE(ctx && ((x && grad_out && grad_in) || n == 0), "hl_gelu_backward: null argument");
  if (n == 0) return HL_OK;
  const bool vec = aligned16(x) && aligned16(grad_out) && aligned16(grad_in);
  if (dtype == HL_F32) {
    map_f32_kernel<<<ew_grid(ctx, vec ? n / 4 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
        (const float*)x, (const float*)grad_out, (float*)grad_in, n, vec,
        [] __device__(float v, float g) { return (float)((double)g * gelu_grad<double>((double)v)); });
  } else if (dtype == HL_BF16) {
    map_bf16_kernel<<<ew_grid(ctx, vec ? n / 8 + 1 : n), EW_THREADS, 0, ctx->stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)grad_out, (__nv_bfloat16*)grad_in, n, vec,
        [] __device__(float v, float g) { return g * gelu_grad_f(v); });
  } else {
    return fail("hl_gelu_backward: dtype must be f32 or bf16");
  }
  HL_LAUNCH_CHECK("gelu backward kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_bias_add_f32(hl_ctx* ctx, const float* x, const float* bias, float* out, int rows, int cols) {
  HL_REQUIRE(ctx && x && bias && out, "hl_bias_add_f32: null argument");
  HL_REQUIRE(rows > 0 && cols > 0, "hl_bias_add_f32: rows and cols must be positive");
  const size_t total = (size_t)rows * cols;
  bias_add_f32_kernel<<<ew_grid(ctx, total), EW_THREADS, 0, ctx->stream>>>(x, bias, out, total, cols);
  HL_LAUNCH_CHECK("bias_add_f32_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_bias_grad(hl_ctx* ctx, const void* grad_out, int dtype, float* grad_bias, int rows, int cols) {
  return bias_grad_impl(ctx, grad_out, dtype, grad_bias, rows, cols);
}

int hl_sum_f32(hl_ctx* ctx, const float* x, size_t n, float* out_dev) { return reduce_impl(ctx, x, n, out_dev, 0, 1.0); }
int hl_mean_f32(hl_ctx* ctx, const float* x, size_t n, float* out_dev) {
  HL_REQUIRE(n > 0, "hl_mean_f32: empty input");
  return reduce_impl(ctx, x, n, out_dev, 0, 1.0 / (double)n);
}
int hl_sum_squares_f32(hl_ctx* ctx, const float* x, size_t n, float* out_dev) {
  return reduce_impl(ctx, x, n, out_dev, 1, 1.0);
}

}  // extern "C"
