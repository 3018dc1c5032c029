// Shared declarations for the sm_100a backend: context, error channel, dtype tags,
// vector helpers.  Everything here is internal; the public surface is include/heirloom_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>
#include <stddef.h>
#include <string>
#include <algorithm>
#include "../../include/heirloom_b200.h"

namespace hl {

// Thread-local UTF-8 message behind hl_last_error(); mirrors the reference's
// CudaError{message} channel (heirloom-kernels/src/cuda.rs:259-280).
void set_error(const std::string& msg);
int fail(const std::string& msg);                      // sets the message, returns HL_ERR_*
int fail_cuda(cudaError_t e, const char* what);

#define HL_CUDA(expr)                                                     \
  do {                                                                    \
    cudaError_t _e = (expr);                                              \
    if (_e != cudaSuccess) return ::hl::fail_cuda(_e, #expr);             \
  } while (0)

#define HL_REQUIRE(cond, msg)                                             \
  do {                                                                    \
    if (!(cond)) return ::hl::fail(std::string(msg));                     \
  } while (0)

#define HL_LAUNCH_CHECK(name)                                             \
  do {                                                                    \
    cudaError_t _e = cudaGetLastError();                                  \
    if (_e != cudaSuccess) return ::hl::fail_cuda(_e, name);              \
  } while (0)

// Device status words.  Kernels never trap: a bad index or an expired wait writes a code
// here and the host folds it into the error channel at the next hl_ctx_sync/hl_status_check
// (the reference reads a status word after each launch, cuda.rs:7184-7193).
enum StatusSlot : int {
  ST_BAD_INDEX = 0,      // out-of-range gather/scatter/target index
  ST_WAIT_EXPIRED = 1,   // a bounded mbarrier wait ran out
  ST_BAD_ARGUMENT = 2,
  ST_SLOTS = 8
};

struct Counters {
  unsigned long long launches, gemm_tcgen05_launches, attention_launches, h2d_bytes, d2h_bytes,
      allocations, allocated_bytes, nccl_calls, nccl_bytes, gemm_pair_launches;
};

}  // namespace hl

struct hl_ctx {
  int device = 0;
  int sm_count = 0;
  unsigned long long wait_limit_ns = 0;  // bound of the pipeline waits in the GEMM kernel (0 = the two-second default)
  int gemm_skip_kblock = -1;           // test hook of hl_ctx_set_test_hooks
  int reserve_sms = 0;                 // SMs the persistent kernels leave free while gradient collectives are in flight
  int comm_sms = 0;                    // how many they leave when asked to (0 = none); set when the communicator is made
  cudaStream_t stream = nullptr;       // compute stream
  cudaStream_t comm_stream = nullptr;  // collective stream
  int* status_dev = nullptr;           // hl::ST_SLOTS ints
  int* status_host = nullptr;          // pinned mirror
  void* workspace = nullptr;           // grow-only scratch (split-K partials, reductions)
  size_t workspace_bytes = 0;
  unsigned* gemm_sched = nullptr;      // counter of the GEMM's dynamic tile order: every processed tile adds one
  unsigned gemm_sched_base = 0;        // its value once every launch queued so far has finished
  void* gemm_flags = nullptr;          // per-CTA hand-over flags of the GEMM's work split, zeroed once
  hl::Counters counters{};
  void* nccl = nullptr;                // hl::NcclState*
  void* profiler = nullptr;            // hl::Profiler*, present while per-kernel timing is on
};

namespace hl {
int ensure_workspace(hl_ctx* ctx, size_t bytes);
inline void count_launch(hl_ctx* ctx, unsigned long long n = 1) { ctx->counters.launches += n; }
// SMs a persistent one-CTA-per-SM kernel should fill: all of them, minus those left to the collective kernels.  A CTA of
// those kernels takes a whole SM's registers or shared memory, so it cannot start on an SM a collective kernel sits
// on, and a grid of one CTA per SM would wait for that SM with its share of the tiles.
inline int persistent_sms(const hl_ctx* ctx) { return std::max(1, ctx->sm_count - ctx->reserve_sms); }

// Opt-in per-kernel timing: a scope brackets the launches of one op with two events on the
// compute stream; hl_profile_read folds them by category after a stream sync (the reference's
// opt-in launch-family timing, heirloom-kernels/src/cuda.rs:8574-8611, forces a sync per
// launch instead).  `work` is the algorithmic flops (GEMM, attention) or bytes (the rest).
void profile_begin(hl_ctx* ctx, int category, double work);
void profile_end(hl_ctx* ctx);
struct ProfileScope {
  hl_ctx* ctx;
  ProfileScope(hl_ctx* c, int category, double work) : ctx(c) { if (c->profiler) profile_begin(c, category, work); }
  ~ProfileScope() { if (ctx->profiler) profile_end(ctx); }
};

inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case HL_F32: return 4;
    case HL_BF16: return 2;
    case HL_F64: return 8;
    case HL_I64: return 8;
    case HL_U8: return 1;
    default: return 0;
  }
}

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

// f32 -> bf16 round-to-nearest-even (same rounding as the reference's storage.rs:440-445).
__device__ __forceinline__ __nv_bfloat16 to_bf16(float x) { return __float2bfloat16_rn(x); }
__device__ __forceinline__ float from_bf16(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

// tanh-approximate GELU and its derivative (reference: src/tensor.rs:5152-5154,
// src/tensor/autograd.rs:2891-2897).
template <typename T>
__device__ __forceinline__ T gelu_fwd(T x) {
  const T c = T(0.7978845608028654);
  T inner = c * (x + T(0.044715) * x * x * x);
  return T(0.5) * x * (T(1) + tanh(inner));
}
template <typename T>
__device__ __forceinline__ T gelu_grad(T x) {
  const T c = T(0.7978845608028654);
  T inner = c * (x + T(0.044715) * x * x * x);
  T t = tanh(inner);
  T sech2 = T(1) - t * t;
  T dinner = c * (T(1) + T(3.0 * 0.044715) * x * x);
  return T(0.5) * (T(1) + t) + T(0.5) * x * sech2 * dinner;
}
__device__ __forceinline__ float gelu_fwd_f(float x) {
  float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t = tanhf(inner);
  float sech2 = 1.0f - t * t;
  float dinner = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
  return 0.5f * (1.0f + t) + 0.5f * x * sech2 * dinner;
}

// Round-to-nearest-even to bf16 precision with integer ops (same result as the conversion
// instruction for every finite input and infinities).  The GEMM epilogues use it because the
// conversion instructions share the 16-lane special-function pipe with tanh.
__device__ __forceinline__ uint32_t bf16_rne_bits(float x) {
  uint32_t u = __float_as_uint(x);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return u & 0xFFFF0000u;
}
__device__ __forceinline__ float bf16_round_alu(float x) { return __uint_as_float(bf16_rne_bits(x)); }
// Packs two floats that are already bf16-representable (low 16 bits zero).
__device__ __forceinline__ uint32_t pack_rounded_bf16x2(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}

// 2^x in one MUFU op (relative error about 2^-22; results below the normal range flush to zero,
// 2^-inf = 0).  exp2f() adds a range check and two scalings around the same instruction.
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Hardware tanh (one MUFU op, relative error about 2^-11): enough for values that are rounded
// to bf16 right after, as in the GEMM epilogues.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The tanh form of GELU and its derivative, written as the shortest chains of fused multiply-adds (the epilogues that use
// them are bound by their instruction count): gelu(x) = hx + hx*t with hx = x/2, t = tanh(x*(k0 + k1*x^2)).
__device__ __forceinline__ float gelu_fwd_fast(float x) {
  constexpr float k0 = 0.7978845608028654f, k1 = 0.7978845608028654f * 0.044715f;
  const float x2 = x * x;
  const float t = tanh_fast(x * fmaf(x2, k1, k0));
  const float hx = 0.5f * x;
  return fmaf(hx, t, hx);
}
// gelu'(x) = (1 + t)/2 + hx*(1 - t^2)*(k0 + 3*k1*x^2)
__device__ __forceinline__ float gelu_grad_fast(float x) {
  constexpr float k0 = 0.7978845608028654f, k1 = 0.7978845608028654f * 0.044715f;
  const float x2 = x * x;
  const float t = tanh_fast(x * fmaf(x2, k1, k0));
  const float dinner = fmaf(x2, 3.0f * k1, k0);
  const float sech2 = fmaf(-t, t, 1.0f);
  return fmaf(0.5f * x * sech2, dinner, fmaf(0.5f, t, 0.5f));
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T>
__device__ __forceinline__ T warp_max(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

// Block-wide sum for blockDim.x <= 1024 (multiple of 32); result valid in every thread.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T* smem /* >= 32 entries */) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  T r = (lane < nw) ? smem[lane] : T(0);
  r = warp_sum(r);
  return r;
}
template <typename T>
__device__ __forceinline__ T block_max(T v, T* smem, T lowest) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  T r = (lane < nw) ? smem[lane] : lowest;
  r = warp_max(r);
  return r;
}

}  // namespace hl
