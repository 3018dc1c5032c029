// Coupled-decay AdamW: single-tensor entry with the reference kernel's exact f32 operation
// order (heirloom-kernels/src/ptx/kernels.ptx:441-467) and a fused multi-tensor launch that
// replaces one launch per parameter (src/nn.rs:2467-2505), optionally writing the bf16 shadow
// weights the next step's GEMMs read.
#include <vector>

#include "common.cuh"

namespace hl {
namespace {

struct AdamChunk {
  float* param;
  const float* grad;
  float* m;
  float* v;
  __nv_bfloat16* shadow;
  unsigned int n;
};

constexpr unsigned int ADAM_CHUNK = 16384;  // elements per block
constexpr int ADAM_THREADS = 256;

// Separately rounded multiply/add/divide/sqrt: identical bits to the reference kernel, which
// has no fused multiply-add.
__device__ __forceinline__ void adamw_element(float& p, float g, float& m, float& v, const hl_adamw_params& hp) {
  const float gd = __fadd_rn(__fmul_rn(g, hp.clip_scale), __fmul_rn(p, hp.weight_decay));
  const float m2 = __fadd_rn(__fmul_rn(hp.beta1, m), __fmul_rn(__fsub_rn(1.0f, hp.beta1), gd));
  const float v2 = __fadd_rn(__fmul_rn(hp.beta2, v), __fmul_rn(__fsub_rn(1.0f, hp.beta2), __fmul_rn(gd, gd)));
  m = m2;
  v = v2;
  const float mh = __fdiv_rn(m2, hp.bias_correction1);
  const float vh = __fdiv_rn(v2, hp.bias_correction2);
  const float upd = __fdiv_rn(mh, __fadd_rn(__fsqrt_rn(vh), hp.eps));
  p = __fsub_rn(p, __fmul_rn(hp.lr, upd));
}

__global__ void __launch_bounds__(ADAM_THREADS)
adamw_chunks_kernel(const AdamChunk* __restrict__ chunks, const hl_adamw_params hp) {
  const AdamChunk ch = chunks[blockIdx.x];
  const unsigned int n4 = ch.n / 4;
  for (unsigned int i = threadIdx.x; i < n4; i += blockDim.x) {
    float4 p = reinterpret_cast<float4*>(ch.param)[i];
    const float4 g = reinterpret_cast<const float4*>(ch.grad)[i];
    float4 m = reinterpret_cast<float4*>(ch.m)[i];
    float4 v = reinterpret_cast<float4*>(ch.v)[i];
    adamw_element(p.x, g.x, m.x, v.x, hp);
    adamw_element(p.y, g.y, m.y, v.y, hp);
    adamw_element(p.z, g.z, m.z, v.z, hp);
    adamw_element(p.w, g.w, m.w, v.w, hp);
    reinterpret_cast<float4*>(ch.param)[i] = p;
    reinterpret_cast<float4*>(ch.m)[i] = m;
    reinterpret_cast<float4*>(ch.v)[i] = v;
    if (ch.shadow)
      reinterpret_cast<uint2*>(ch.shadow)[i] = make_uint2(pack_bf16x2(p.x, p.y), pack_bf16x2(p.z, p.w));
  }
  for (unsigned int i = n4 * 4 + threadIdx.x; i < ch.n; i += blockDim.x) {
    float p = ch.param[i], m = ch.m[i], v = ch.v[i];
    adamw_element(p, ch.grad[i], m, v, hp);
    ch.param[i] = p; ch.m[i] = m; ch.v[i] = v;
    if (ch.shadow) ch.shadow[i] = to_bf16(p);
  }
}

__global__ void adamw_scalar_kernel(float* __restrict__ param, const float* __restrict__ grad, float* __restrict__ m,
                                    float* __restrict__ v, size_t n, const hl_adamw_params hp) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = tid; i < n; i += stride) {
    float p = param[i], mm = m[i], vv = v[i];
    adamw_element(p, grad[i], mm, vv, hp);
    param[i] = p; m[i] = mm; v[i] = vv;
  }
}

int validate(const hl_adamw_params* hp, const char* who) {
  HL_REQUIRE(hp != nullptr, std::string(who) + ": null hyper-parameters");
  HL_REQUIRE(hp->bias_correction1 > 0.f && hp->bias_correction2 > 0.f,
             std::string(who) + ": bias corrections must be positive (step >= 1)");
  return HL_OK;
}

}  // namespace

// A reusable chunk table on the device.  Built once per parameter set by the step executor.
struct AdamPlan {
  AdamChunk* chunks_dev = nullptr;
  int count = 0;
  unsigned long long elements = 0;
};

int adam_plan_create(hl_ctx* ctx, const hl_adamw_tensor* tensors, int count, AdamPlan** out) {
  HL_REQUIRE(ctx && tensors && out && count > 0, "adamw plan: null or empty argument");
  std::vector<AdamChunk> chunks;
  unsigned long long elements_total = 0;
  for (int t = 0; t < count; ++t) {
    const hl_adamw_tensor& x = tensors[t];
    HL_REQUIRE(x.param && x.grad && x.m && x.v, "adamw plan: null tensor pointer");
    HL_REQUIRE(((reinterpret_cast<uintptr_t>(x.param) | reinterpret_cast<uintptr_t>(x.grad) |
                 reinterpret_cast<uintptr_t>(x.m) | reinterpret_cast<uintptr_t>(x.v)) & 15) == 0,
               "adamw plan: tensors must be 16-byte aligned");
    HL_REQUIRE(!x.shadow_bf16 || (reinterpret_cast<uintptr_t>(x.shadow_bf16) & 7) == 0,
               "adamw plan: bf16 shadow must be 8-byte aligned");
    for (uint64_t off = 0; off < x.n; off += ADAM_CHUNK) {
      AdamChunk c;
      c.param = x.param + off; c.grad = x.grad + off; c.m = x.m + off; c.v = x.v + off;
      c.shadow = x.shadow_bf16 ? reinterpret_cast<__nv_bfloat16*>(x.shadow_bf16) + off : nullptr;
      c.n = (unsigned int)std::min<uint64_t>(ADAM_CHUNK, x.n - off);
      chunks.push_back(c);
    }
    elements_total += x.n;
  }
  AdamPlan* plan = new AdamPlan();
  plan->count = (int)chunks.size();
  plan->elements = elements_total;
  if (plan->count > 0) {
    cudaError_t e = cudaMalloc(&plan->chunks_dev, sizeof(AdamChunk) * chunks.size());
    if (e != cudaSuccess) { delete plan; return fail_cuda(e, "cudaMalloc(adamw chunk table)"); }
    e = cudaMemcpyAsync(plan->chunks_dev, chunks.data(), sizeof(AdamChunk) * chunks.size(), cudaMemcpyHostToDevice,
                        ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { cudaFree(plan->chunks_dev); delete plan; return fail_cuda(e, "upload adamw chunk table"); }
  }
  *out = plan;
  return HL_OK;
}

void adam_plan_destroy(AdamPlan* plan) {
  if (!plan) return;
  if (plan->chunks_dev) cudaFree(plan->chunks_dev);
  delete plan;
}

int adam_plan_chunk_elements() { return (int)ADAM_CHUNK; }
int adam_plan_chunk_count(const AdamPlan* plan) { return plan->count; }

// Chunks [first, first + count) of the table: lets a caller update the part of a gradient arena whose
// all-reduce has finished while the rest is still in flight.
int adam_plan_step_range(hl_ctx* ctx, AdamPlan* plan, const hl_adamw_params* hp, int first, int count) {
  int rc = validate(hp, "hl_adamw_multi");
  if (rc != HL_OK) return rc;
  HL_REQUIRE(first >= 0 && count >= 0 && first + count <= plan->count, "adamw plan: chunk range out of bounds");
  if (count == 0) return HL_OK;
  // 28 bytes per parameter (read p, g, m, v; write p, m, v) plus 2 for the bf16 shadow
  ProfileScope prof(ctx, HL_PROF_OPTIMIZER, 30.0 * (double)plan->elements * ((double)count / (double)plan->count));
  adamw_chunks_kernel<<<count, ADAM_THREADS, 0, ctx->stream>>>(plan->chunks_dev + first, *hp);
  HL_LAUNCH_CHECK("adamw_chunks_kernel");
  count_launch(ctx);
  return HL_OK;
}

int adam_plan_step(hl_ctx* ctx, AdamPlan* plan, const hl_adamw_params* hp) {
  return adam_plan_step_range(ctx, plan, hp, 0, plan->count);
}

}  // namespace hl

using namespace hl;

extern "C" {

int hl_adamw_f32(hl_ctx* ctx, float* param, const float* grad, float* m, float* v, size_t n, const hl_adamw_params* hp) {
  HL_REQUIRE(ctx && ((param && grad && m && v) || n == 0), "hl_adamw_f32: null argument");
  int rc = validate(hp, "hl_adamw_f32");
  if (rc != HL_OK) return rc;
  if (n == 0) return HL_OK;
  const int grid = (int)std::min<size_t>((n + 255) / 256, (size_t)ctx->sm_count * 16);
  adamw_scalar_kernel<<<grid, 256, 0, ctx->stream>>>(param, grad, m, v, n, *hp);
  HL_LAUNCH_CHECK("adamw_scalar_kernel");
  count_launch(ctx);
  return HL_OK;
}

int hl_adamw_multi(hl_ctx* ctx, const hl_adamw_tensor* tensors_host, int count, const hl_adamw_params* hp) {
  AdamPlan* plan = nullptr;
  int rc = adam_plan_create(ctx, tensors_host, count, &plan);
  if (rc != HL_OK) return rc;
  rc = adam_plan_step(ctx, plan, hp);
  if (rc == HL_OK) {
    cudaError_t e = cudaStreamSynchronize(ctx->stream);  // the table is freed right after
    if (e != cudaSuccess) rc = fail_cuda(e, "cudaStreamSynchronize");
  }
  adam_plan_destroy(plan);
  return rc;
}

int hl_adamw_plan_create(hl_ctx* ctx, const hl_adamw_tensor* tensors_host, int count, hl_adamw_plan** out) {
  HL_REQUIRE(out, "hl_adamw_plan_create: null output pointer");
  *out = nullptr;
  AdamPlan* plan = nullptr;
  int rc = adam_plan_create(ctx, tensors_host, count, &plan);
  if (rc == HL_OK) *out = reinterpret_cast<hl_adamw_plan*>(plan);
  return rc;
}

int hl_adamw_plan_step(hl_ctx* ctx, hl_adamw_plan* plan, const hl_adamw_params* hp) {
  HL_REQUIRE(ctx && plan, "hl_adamw_plan_step: null argument");
  return adam_plan_step(ctx, reinterpret_cast<AdamPlan*>(plan), hp);
}

void hl_adamw_plan_destroy(hl_adamw_plan* plan) { adam_plan_destroy(reinterpret_cast<AdamPlan*>(plan)); }

}  // extern "C"
