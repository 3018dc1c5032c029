// Internal entry points shared between translation units: the same kernels the C ABI exposes,
// with scratch memory passed explicitly so the step executor can plan it once.
#pragma once
#include "common.cuh"

namespace hl {

// How a GEMM's work is cut: explicit split-K (partial sums for a second kernel), or whole waves of
// tiles followed by tiles whose k blocks are dealt out evenly over the CTAs.
struct GemmPlan {
  int splits;
  int dp_tiles, sk_tiles;
  size_t splitk_bytes;   // scratch for explicit split-K partial sums
  size_t sk_slot_bytes;  // scratch for the raw accumulators of partly finished tiles
};
GemmPlan gemm_plan(const hl_gemm_desc* d, int sm_count);
int gemm_bf16_run(hl_ctx* ctx, const hl_gemm_desc* d, const void* a, const void* b, void* c, const float* bias,
                  const void* aux_in, void* aux_out, float* workspace, size_t workspace_bytes, unsigned* stream_flags);
// The GEMM with its scratch taken from (and grown in) the context.
int gemm_bf16_ctx(hl_ctx* ctx, const hl_gemm_desc* d, const void* a, const void* b, void* c, const float* bias,
                  const void* aux_in, void* aux_out);

// Column reductions (layer-norm parameter gradients, bias gradients) end in a fold of per-block partial rows.  A
// caller that runs several of them before anyone reads the results hands in a FoldBatch: the kernels then leave their
// partial rows in the batch's scratch and one launch (fold_batch_flush) folds all of them, in a fixed order.
struct FoldJob {
  const float* partial;  // [blocks][total]
  int blocks, total, features;
  float *o0, *o1, *o2;   // column c goes to o(c / features)[c % features]; null outputs are skipped
};
struct FoldBatch {
  static constexpr int kMaxJobs = 8;
  FoldJob jobs[kMaxJobs];
  int n = 0;
  float* scratch = nullptr;  // device memory, `capacity` floats
  size_t capacity = 0, used = 0;
};
// Room for `elems` partial sums in the batch, or null when the batch is absent or full (the caller then folds at once).
float* fold_batch_reserve(FoldBatch* batch, size_t elems);
void fold_batch_add(FoldBatch* batch, const float* partial, int blocks, int total, int features, float* o0, float* o1,
                    float* o2);
int fold_batch_flush(hl_ctx* ctx, FoldBatch* batch);

int bias_grad_impl(hl_ctx* ctx, const void* grad_out, int dtype, float* grad_bias, int rows, int cols,
                   FoldBatch* defer = nullptr);

int layer_norm_forward_impl(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* beta, void* y,
                            int y_dtype, float* mean, float* rstd, int rows, int features, float eps);
int layer_norm_backward_impl(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* dy,
                             const float* mean, const float* rstd, const float* residual_grad, float* dx_f32,
                             void* dx_bf16, float* dgamma, float* dbeta, float* dx_colsum, int rows, int features,
                             FoldBatch* defer = nullptr);
bool layer_norm_fast_applicable(int x_dtype, int y_dtype, int features, const void* x, const void* y);
int layer_norm_forward_fast(hl_ctx* ctx, const void* x, const float* gamma, const float* beta, void* y, float* mean,
                            float* rstd, int rows, int features, float eps);
int layer_norm_backward_fast(hl_ctx* ctx, const void* x, const float* gamma, const float* dy, const float* mean,
                             const float* rstd, const float* residual, float* dx_f32, void* dx_bf16, float* dgamma,
                             float* dbeta, float* dx_colsum, int rows, int features, FoldBatch* defer = nullptr);
bool colsum_fast_applicable(int dtype, int cols, const void* g);
int colsum_fast(hl_ctx* ctx, const void* g, int dtype, float* out, int rows, int cols, FoldBatch* defer = nullptr);
int cross_entropy_impl(hl_ctx* ctx, const float* logits, long long ld, const int64_t* targets, int rows, int classes,
                       float grad_scale, float* loss_dev, float* row_loss, void* dlogits, int dlogits_dtype,
                       long long ld_dlogits);

int flash_attention_forward_impl(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv, void* out,
                                 long long ld_out, float* lse, int batch, int time, int n_heads, int head_dim);
size_t flash_attention_backward_scratch_bytes(int batch, int time, int n_heads, int head_dim);
int flash_attention_backward_impl(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv,
                                  const void* out, long long ld_out, const void* dout, long long ld_dout,
                                  const float* lse, void* dq, void* dk, void* dv, long long ld_dqkv, int batch, int time,
                                  int n_heads, int head_dim, void* scratch, size_t scratch_bytes);

struct AdamPlan;
int adam_plan_create(hl_ctx* ctx, const hl_adamw_tensor* tensors, int count, AdamPlan** out);
void adam_plan_destroy(AdamPlan* plan);
int adam_plan_step(hl_ctx* ctx, AdamPlan* plan, const hl_adamw_params* hp);
int adam_plan_step_range(hl_ctx* ctx, AdamPlan* plan, const hl_adamw_params* hp, int first, int count);
int adam_plan_chunk_elements();
int adam_plan_chunk_count(const AdamPlan* plan);

extern "C" int hl_memory_copy_indices(hl_ctx* ctx, int64_t* host, const int64_t* dev, long long count);

// NCCL (loaded at run time); see nccl_ddp.cu.
int nccl_allreduce_sum_f32(hl_ctx* ctx, float* buf, size_t count, cudaStream_t stream);
int nccl_allreduce_max_u8(hl_ctx* ctx, unsigned char* buf, size_t count, cudaStream_t stream);
int mark_rows_on(hl_ctx* ctx, cudaStream_t stream, const int64_t* selected_rows, long long n_selected, const unsigned char* row_mask,
                 unsigned char* flags, int rows);
int mask_to_indices_on(hl_ctx* ctx, cudaStream_t stream, const unsigned char* mask, int rows, int64_t* out, int* count_dev);
int move_rows_on(hl_ctx* ctx, cudaStream_t stream, const float* src, const int64_t* idx, const int* count_dev, int n_max, int dim,
                 float* dst, bool scatter);
bool nccl_active(const hl_ctx* ctx);
int nccl_world(const hl_ctx* ctx);

}  // namespace hl
