/*
 * heirloom_b200 — C ABI of the sm_100a backend for Heirloom's transformer training step.
 *
 * Every entry point returns 0 (HL_OK) or a negative HL_ERR_* code; the message is available
 * from hl_last_error() (thread local).  Nothing throws or aborts across this boundary.
 * Pointers named `*_dev` / documented as device pointers are plain CUDA device addresses;
 * sizes are element counts unless they say bytes.  No kernel traps on bad data: device-side
 * problems (out-of-range index, expired wait) are written to status words that
 * hl_ctx_sync()/hl_status_check() fold into the same error channel.
 *
 * File:line citations name the reference interface each entry point replaces, by path inside
 * the Heirloom repository.
 */
#ifndef HEIRLOOM_B200_H
#define HEIRLOOM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HL_OK 0
#define HL_ERR_INVALID (-1) /* argument validation failed before any launch */
#define HL_ERR_CUDA (-2)    /* a CUDA runtime/driver call failed */
#define HL_ERR_DEVICE (-3)  /* a kernel reported a problem through the status words */
#define HL_ERR_NCCL (-4)

/* Element types (reference: DType, src/storage.rs:14-20; device bool is one byte). */
enum { HL_F32 = 0, HL_BF16 = 1, HL_F64 = 2, HL_I64 = 3, HL_U8 = 4 };

typedef struct hl_ctx hl_ctx;
typedef struct hl_buffer hl_buffer;

/* ---- runtime -------------------------------------------------------------------------------
 * One context per (thread, device): one compute stream and one collective stream, a status
 * buffer and a grow-only scratch arena.  Replaces the per-thread context/stream cache of
 * heirloom-kernels/src/cuda.rs:7517-7521, :7653-7681.  Not thread-safe by contract. */
int hl_ctx_create(int device_ordinal, hl_ctx** out);
void hl_ctx_destroy(hl_ctx* ctx);
/* Waits for the compute stream, then reports any device status word as an error. */
int hl_ctx_sync(hl_ctx* ctx);
/* Test hooks of the failure path.  Every wait inside the tcgen05 kernels is bounded (two seconds by default): when a
 * wait runs out the kernel leaves its loops, frees its tensor memory, returns, and sets a status word that the next
 * hl_ctx_sync reports as HL_ERR_DEVICE; the context stays usable.  `wait_limit_ns` shortens the bound for hl_gemm_bf16
 * (0 = default) and `gemm_skip_kblock` >= 0 makes the GEMM's TMA producer leave out that k block of its first tile,
 * so that the wait for it runs out; -1 switches the hook off.  The reference has no such path: its kernels have no
 * device-side waits (single-role kernels, heirloom-kernels/src/ptx/tensor_core.ptx). */
int hl_ctx_set_test_hooks(hl_ctx* ctx, unsigned long long wait_limit_ns, int gemm_skip_kblock);
/* The compute stream as a cudaStream_t, for callers that time with their own events. */
void* hl_ctx_stream(hl_ctx* ctx);
const char* hl_last_error(void);
/* FNV-1a, 64 bit, continued from `seed` (0xcbf29ce484222325 to start): the hash the reference
 * records for token shards and their payload files (src/tokenizer.rs:968-975, src/data.rs:1979-2005).
 * Host function, no device work. */
unsigned long long hl_fnv1a64(const void* data, size_t bytes, unsigned long long seed);

/* Device facts (reference: device_supports_bf16_tensor_cores, cuda.rs:8290-8296). */
typedef struct {
  int sm_major, sm_minor, sm_count;
  size_t total_bytes, free_bytes;
  int supports_tcgen05; /* 1 only on compute capability 10.x */
} hl_device_info_t;
int hl_device_info(hl_ctx* ctx, hl_device_info_t* out);

/* Counters (reference: cuda_runtime_counters / tensor_core_counters, cuda.rs:1589-2014). */
typedef struct {
  uint64_t launches, gemm_tcgen05_launches, attention_launches, h2d_bytes, d2h_bytes, allocations,
      allocated_bytes, nccl_calls, nccl_bytes,
      gemm_pair_launches; /* those of gemm_tcgen05_launches that ran on pairs of CTAs (256-row tiles) */
} hl_counters_t;
int hl_counters_get(hl_ctx* ctx, hl_counters_t* out);
int hl_counters_reset(hl_ctx* ctx);

/* Opt-in per-kernel timing with CUDA events on the compute stream, folded by category
 * (reference: launch-family timing, cuda.rs:8574-8611, and CudaEventTimer, :853-949).
 * `work` is algorithmic flops for GEMM/attention categories and bytes for the others. */
enum {
  HL_PROF_GEMM = 0, HL_PROF_ATTENTION_FWD = 1, HL_PROF_ATTENTION_BWD = 2, HL_PROF_LAYER_NORM = 3, HL_PROF_LOSS = 4,
  HL_PROF_OPTIMIZER = 5, HL_PROF_BIAS_GRAD = 6, HL_PROF_EMBEDDING = 7, HL_PROF_OTHER = 8, HL_PROF_CATEGORIES = 9
};
typedef struct {
  double ms[HL_PROF_CATEGORIES];
  double work[HL_PROF_CATEGORIES];
  uint64_t scopes[HL_PROF_CATEGORIES];
} hl_profile_t;
int hl_profile_enable(hl_ctx* ctx, int on);
int hl_profile_read(hl_ctx* ctx, hl_profile_t* out);

/* Reference-counted device buffers (reference: CudaBuffer, cuda.rs:652-656; frees are
 * stream-ordered as in :7870-7922).  hl_memcpy_d2h waits for the compute stream first
 * (cuda.rs:836). */
int hl_buffer_alloc(hl_ctx* ctx, size_t bytes, hl_buffer** out);
int hl_buffer_retain(hl_buffer* buf);
int hl_buffer_release(hl_buffer* buf);
void* hl_buffer_ptr(hl_buffer* buf);
size_t hl_buffer_bytes(hl_buffer* buf);
int hl_memcpy_h2d(hl_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int hl_memcpy_d2h(hl_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
int hl_memset_zero(hl_ctx* ctx, void* dst_dev, size_t bytes);

/* ---- elementwise ---------------------------------------------------------------------------
 * f32 add/sub/mul/div (reference: heirloom_add/sub/mul/div_f32, kernels.ptx:6-141). */
enum { HL_ADD = 0, HL_SUB = 1, HL_MUL = 2, HL_DIV = 3 };
int hl_binary_f32(hl_ctx* ctx, int op, const float* a, const float* b, float* out, size_t n);
/* out = a * s (kernels.ptx:142). */
int hl_scale_f32(hl_ctx* ctx, const float* a, float s, float* out, size_t n);
/* kernels.ptx:1131. */
int hl_fill_f32(hl_ctx* ctx, float* out, float value, size_t n);
/* Plain SGD, param -= lr * grad with the product and the difference rounded separately; lr must be positive
 * (sgd_update_f32_buffer, heirloom-kernels/src/cuda.rs:6280-6303; heirloom_sgd_update_f32, kernels.ptx:356). */
int hl_sgd_update_f32(hl_ctx* ctx, float* param, const float* grad, float lr, size_t n);
/* out[i] = i (i64_arange_buffer, cuda.rs:2090-2103; heirloom_i64_arange, kernels.ptx:861): the position ids of the
 * learned position embedding. */
int hl_arange_i64(hl_ctx* ctx, int64_t* out, size_t n);
/* The inputs one after the other in `out` (concat_i64_buffers, cuda.rs:6437-6490; heirloom_copy_i64_with_offset,
 * kernels.ptx:1066): how the selected rows of several memory blocks become one row list for the row-set AdamW.
 * Empty inputs are skipped; `out_capacity` is checked against the summed lengths before anything is launched. */
int hl_concat_i64(hl_ctx* ctx, const int64_t* const* inputs, const size_t* lengths, int count, int64_t* out,
                  size_t out_capacity);
/* ReLU and its gradient (kernels.ptx:4724, :4755). */
int hl_relu_f32(hl_ctx* ctx, const float* x, float* out, size_t n);
int hl_relu_backward_f32(hl_ctx* ctx, const float* x, const float* grad_out, float* grad_in, size_t n);
/* Casts with round-to-nearest-even (kernels.ptx:174, :208, :238; src/storage.rs:440-449).
 * src_dtype/dst_dtype in {HL_F32, HL_BF16}; equal f32 types perform the bf16 round trip. */
int hl_cast(hl_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, size_t n);
/* An f32 matrix [rows, cols] as bf16 pieces laid side by side along the columns, dst [rows, pieces*cols]:
 * hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid) (the differences are exact).  With them a product
 * with an f32 operand runs on the bf16 tensor cores at f32 accuracy (hl_gemm_desc.a_k_period): this is how the
 * memory feed-forward keeps its projections in f32 under AMP, as the reference does
 * (src/memory_transformer.rs:787-789), without leaving the tensor cores.
 *   HL_SPLIT_HI_MID_LO  [hi | mid | lo]   exact three-piece form of a weight, against a bf16-exact input
 *   HL_SPLIT_HI_HI_LO   [hi | hi | mid]   weight side of hi*hi + lo*hi + hi*lo
 *   HL_SPLIT_HI_LO      [hi | mid]        input side of the same, read with a_k_period = 2*cols */
enum { HL_SPLIT_HI_MID_LO = 0, HL_SPLIT_HI_HI_LO = 1, HL_SPLIT_HI_LO = 2,
       HL_SPLIT_STACK_ROWS = 4 /* or-ed in: the pieces one below the other, dst [pieces*rows, cols], for operands whose
                                  rows are the contraction index */ };
int hl_split_bf16_f32(hl_ctx* ctx, const float* src, void* dst, long long rows, int cols, int mode);
/* tanh-GELU and its gradient (kernels.ptx:4791, :4842; src/tensor.rs:5152-5154,
 * src/tensor/autograd.rs:2891-2897).  dtype in {HL_F32, HL_BF16} applies to x/out/grads. */
int hl_gelu(hl_ctx* ctx, const void* x, void* out, int dtype, size_t n);
int hl_gelu_backward(hl_ctx* ctx, const void* x, const void* grad_out, void* grad_in, int dtype, size_t n);
/* out[r,c] = x[r,c] + bias[c] (kernels.ptx:272). */
int hl_bias_add_f32(hl_ctx* ctx, const float* x, const float* bias, float* out, int rows, int cols);
/* Column sums: grad_bias[c] = sum_r grad_out[r,c] (kernels.ptx:312).  grad_out dtype f32 or
 * bf16, f32 result; a two-stage reduction instead of one serial thread per column. */
int hl_bias_grad(hl_ctx* ctx, const void* grad_out, int dtype, float* grad_bias, int rows, int cols);

/* ---- reductions (kernels.ptx:4610, :4647, :4685): result is one f32 on the device ---------- */
int hl_sum_f32(hl_ctx* ctx, const float* x, size_t n, float* out_dev);
int hl_mean_f32(hl_ctx* ctx, const float* x, size_t n, float* out_dev);
int hl_sum_squares_f32(hl_ctx* ctx, const float* x, size_t n, float* out_dev);

/* ---- layer norm over the last dimension ----------------------------------------------------
 * Forward (reference: src/tensor.rs:3175-3256, kernels.ptx:3260): biased variance,
 * rstd = 1/sqrt(var+eps).  x/y dtypes in {HL_F32, HL_BF16}; gamma/beta f32; saves per-row
 * mean and rstd (f32, may be NULL). */
int hl_layer_norm_forward(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* beta,
                          void* y, int y_dtype, float* mean, float* rstd, int rows, int features, float eps);
/* Backward (src/tensor/autograd.rs:2158-2232, kernels.ptx:3347, :3463):
 *   dx = rstd*(F*dxhat - sum(dxhat) - xhat*sum(dxhat*xhat))/F  [+ residual_grad if given]
 *   dgamma = sum_rows dy*xhat, dbeta = sum_rows dy.
 * dy and residual_grad are f32; dx is written as f32 (dx_f32) and/or bf16 (dx_bf16), either
 * may be NULL.  mean/rstd as saved by the forward.  dx_colsum (may be NULL) receives the column
 * sums of the dx written, i.e. the bias gradient of the linear layer whose output this layer
 * norm consumed (the reference computes it with a separate kernel, kernels.ptx:312). */
int hl_layer_norm_backward(hl_ctx* ctx, const void* x, int x_dtype, const float* gamma, const float* dy,
                           const float* mean, const float* rstd, const float* residual_grad, float* dx_f32,
                           void* dx_bf16, float* dgamma, float* dbeta, float* dx_colsum, int rows, int features);

/* ---- embedding -----------------------------------------------------------------------------
 * out[n,:] = table[idx[n],:] (+ pos_table[n % period,:] when pos_table != NULL, each term and
 * the sum rounded to out_dtype as the reference's AMP route does, memory_transformer.rs:1636-1648).
 * (reference: src/tensor.rs:3337-3395, kernels.ptx:1660).  Out-of-range ids set a status word. */
int hl_embedding_forward(hl_ctx* ctx, const float* table, int table_rows, const int64_t* idx,
                         const float* pos_table, int period, void* out, int out_dtype, int n, int dim);
/* grad_table[idx[n],:] += grad_out[n,:]; repeats accumulate (src/tensor/autograd.rs:2234-2261,
 * kernels.ptx:1720).  grad_table must be zeroed by the caller when it starts a new step.
 * When pos_grad != NULL also pos_grad[n % period,:] += grad_out[n,:]. */
int hl_embedding_backward(hl_ctx* ctx, const float* grad_out, const int64_t* idx, float* grad_table,
                          int table_rows, float* pos_grad, int period, int n, int dim);

/* ---- softmax cross-entropy with fused logits gradient --------------------------------------
 * loss = mean_rows(-z[y] + max + ln sum exp(z - max)) (src/tensor.rs:4816-4882,
 * kernels.ptx:3558); dlogits = (softmax - onehot) * grad_scale / rows
 * (src/tensor/autograd.rs:2591-2621, kernels.ptx:3658).  logits f32 `[rows, classes]` with row
 * stride `ld`; dlogits (may be NULL) f32 or bf16, may alias logits when f32.  row_loss (may be
 * NULL) receives per-row losses; loss_dev receives the mean. */
int hl_cross_entropy(hl_ctx* ctx, const float* logits, long long ld, const int64_t* targets, int rows,
                     int classes, float grad_scale, float* loss_dev, float* row_loss, void* dlogits,
                     int dlogits_dtype, long long ld_dlogits);

/* ---- coupled-decay AdamW -------------------------------------------------------------------
 * Arithmetic and operation order of the reference kernel (kernels.ptx:441-467; host side
 * src/nn.rs:2156-2220): g' = g*clip + wd*p; m = b1*m + (1-b1)*g'; v = b2*v + (1-b2)*g'*g';
 * p -= lr * (m/bc1) / (sqrt(v/bc2) + eps), every product and sum rounded separately. */
typedef struct {
  float lr, beta1, beta2, eps, weight_decay, clip_scale, bias_correction1, bias_correction2;
} hl_adamw_params;
int hl_adamw_f32(hl_ctx* ctx, float* param, const float* grad, float* m, float* v, size_t n,
                 const hl_adamw_params* hp);
/* One launch over many tensors (replaces one launch per parameter, src/nn.rs:2467-2505).
 * Each entry is a 16-byte aligned chunk of one tensor; `shadow_bf16` (may be NULL) receives
 * the updated parameter rounded to bf16 for the next step's GEMM operands. */
typedef struct {
  float* param;
  const float* grad;
  float* m;
  float* v;
  void* shadow_bf16;
  uint64_t n;
} hl_adamw_tensor;
int hl_adamw_multi(hl_ctx* ctx, const hl_adamw_tensor* tensors_host, int count, const hl_adamw_params* hp);
/* The same update with the tensor table built once: an optimizer owns a plan for its parameter set and
 * steps it every iteration with that iteration's hyper-parameters (hl_adamw_multi builds and frees a table
 * on every call, which costs a device allocation).  The plan keeps pointers, not data. */
typedef struct hl_adamw_plan hl_adamw_plan;
int hl_adamw_plan_create(hl_ctx* ctx, const hl_adamw_tensor* tensors_host, int count, hl_adamw_plan** out);
int hl_adamw_plan_step(hl_ctx* ctx, hl_adamw_plan* plan, const hl_adamw_params* hp);
void hl_adamw_plan_destroy(hl_adamw_plan* plan);

/* ---- GEMM ----------------------------------------------------------------------------------
 * f32 strided matmul with f64 accumulation: out[i,j] = sum_k A[i,k]*B[k,j] with arbitrary
 * element strides and offsets (reference: heirloom_matmul_f32_strided, kernels.ptx:1455-1659;
 * MatrixLayout, cuda.rs:536-560).  Used by the f32 parity mode; not a throughput path. */
typedef struct {
  long long rows, cols, row_stride, col_stride, offset;
} hl_matrix_layout;
int hl_matmul_f32_strided(hl_ctx* ctx, const float* a, const hl_matrix_layout* la, const float* b,
                          const hl_matrix_layout* lb, float* out, const hl_matrix_layout* lo, int accumulate);

/* ---- causal self-attention, f32 route -------------------------------------------------------
 * q, k, v, out: [batch, time, channels] with heads interleaved along channels
 * (index b*T*C + t*C + h*hd + j, src/tensor.rs:5156-5177); scale 1/sqrt(hd); probs
 * [batch, heads, time, time] is saved for the backward like the reference's f32 CUDA route
 * (src/tensor.rs:3980-4098, :4404-4494; kernels.ptx:3760-4609).  f64 accumulation. */
int hl_causal_attention_f32_forward(hl_ctx* ctx, const float* q, const float* k, const float* v, float* out,
                                    float* probs, int batch, int time, int channels, int n_heads);
/* dQ, dK, dV from the saved probabilities (src/tensor/autograd.rs:2623-2712); sums run in a
 * fixed order (no atomics). */
int hl_causal_attention_f32_backward(hl_ctx* ctx, const float* q, const float* k, const float* v,
                                     const float* probs, const float* grad_out, float* dq, float* dk, float* dv,
                                     int batch, int time, int channels, int n_heads);

/* bf16 x bf16 -> f32-accumulate GEMM on tcgen05 tensor cores:
 *   C[m,n] = A[m,k] * B[k,n] with operand storage chosen per side,
 *   a_layout: HL_K_MAJOR  A stored [m][k] (k contiguous, row stride lda)
 *             HL_MN_MAJOR A stored [k][m] (m contiguous, row stride lda)
 *   b_layout: HL_K_MAJOR  B stored [n][k] (k contiguous, row stride ldb)  -- "rhs_t"
 *             HL_MN_MAJOR B stored [k][n] (n contiguous, row stride ldb)  -- "normal rhs"
 * so forward (X*W^T), dgrad (dY*W) and wgrad (dY^T*X) need no transpose or pad kernels.
 * Replaces matmul_bf16_tensor_core_* (cuda.rs:4215-4386; tensor_core.ptx:42-1527) and the
 * bias / cast / gelu kernels around them.  Epilogues act on the f32 accumulator:
 *   HL_EPI_NONE           C = acc
 *   HL_EPI_BIAS           C = acc + bias[n]
 *   HL_EPI_BIAS_GELU      C = bf16(acc + bias) and aux_out = bf16(gelu(C))
 *   HL_EPI_BIAS_RESIDUAL  C = bf16(aux_in + bf16(acc + bias))
 *   HL_EPI_DGELU          C = acc * gelu'(aux_in)
 * Requirements: n, lda, ldb, ldc multiples of 8; 16-byte aligned pointers.  split_k = 0 lets
 * the library split the contraction for small outputs (plain f32 output only; partial sums go
 * through the context's scratch arena and are reduced in a fixed order). */
enum { HL_K_MAJOR = 0, HL_MN_MAJOR = 1 };
enum { HL_EPI_NONE = 0, HL_EPI_BIAS = 1, HL_EPI_BIAS_GELU = 2, HL_EPI_BIAS_RESIDUAL = 3, HL_EPI_DGELU = 4 };
typedef struct {
  int m, n, k;
  int a_layout, b_layout;
  long long lda, ldb, ldc;
  int epilogue;
  int out_dtype; /* HL_BF16 or HL_F32 */
  int split_k;
  long long ld_aux_in, ld_aux_out; /* 0 = same as ldc */
  int a_k_period; /* 0, or a multiple of 64: A holds only this many contraction elements and is read again
                     from its start after them (B supplies all k), so that one f32 accumulation can take
                     C = A*B1 + A*B2 + ... with B = [B1 | B2 | ...] along the contraction */
  int b_k_period; /* the same for B */
} hl_gemm_desc;
int hl_gemm_bf16(hl_ctx* ctx, const hl_gemm_desc* desc, const void* a, const void* b, void* c,
                 const float* bias, const void* aux_in, void* aux_out);

/* How hl_gemm_bf16 would cut this shape on this context's GPU: the number of equal splits of the contraction
 * (1 = none), the number of output tiles whose k blocks are dealt out over the CTAs (0 = none), and the scratch
 * bytes the launch needs.  Pure host arithmetic; lets a caller check a shape against a scratch budget before the
 * step starts (the reference's shape-support predicates play this role, heirloom-kernels/src/cuda.rs:3761-3900). */
int hl_gemm_bf16_plan(hl_ctx* ctx, const hl_gemm_desc* desc, int* splits, int* dealt_tiles, size_t* scratch_bytes);

/* The same GEMM for callers that must not allocate.  It has no counterpart in the reference.
 * hl_gemm_bf16 keeps split-K partial sums in the context's scratch arena and grows that arena
 * with the CUDA allocator when needed; a host runtime that has given all free device memory to
 * its own pool, or a step loop whose compute and collective streams are overlapped (an allocator
 * call may wait for the whole device), cannot afford that.  Here the partial sums live in a
 * fixed 32 MiB array inside the library image, held by every GPU that loads the library until
 * the process exits.  Shapes whose split-K scratch (splits * m * n * 4 bytes) exceeds 32 MiB are
 * rejected with an error; nothing is allocated, freed or resized by this call.  The first call
 * on a device looks up the array's device address (make that call before starting any stream
 * capture).  All calls share the array and it keeps the previous call's contents (a split-K
 * launch overwrites everything it later reads, so nothing needs clearing); two calls that
 * overlap on the GPU, e.g. from two contexts on one device, race on it.  Per-kernel timing must
 * be off.  Arguments and results are those of hl_gemm_bf16. */
int hl_gemm_bf16_static_scratch(hl_ctx* ctx, const hl_gemm_desc* desc, const void* a, const void* b, void* c,
                                const float* bias, const void* aux_in, void* aux_out);

/* ---- causal flash attention, bf16 route ----------------------------------------------------
 * q, k, v: bf16 row-major views of [batch*time, *] with row stride ld_qkv and heads interleaved
 * along the channel dimension (column h*head_dim + j, src/tensor.rs:5156-5177), so the three
 * may be column slices of one fused projection buffer.  out: bf16 [batch*time, heads*head_dim]
 * with row stride ld_out.  lse: f32 [batch, heads, time], natural-log log-sum-exp of the scaled
 * scores, saved for the backward (the reference saves row_max and row_denom instead,
 * src/tensor.rs:4164-4358).  P enters the PV product rounded to bf16, accumulation is f32.
 * Replaces causal_attention_bf16_flash_tensor_core_forward_f32_buffers (cuda.rs:5283-5420,
 * tensor_core.ptx:2284-2981, which takes any head_dim that is a multiple of 16).  head_dim must be 64 or 128;
 * wider heads are handled as 64-channel blocks side by side. */
int hl_flash_attention_forward(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv,
                               void* out, long long ld_out, float* lse, int batch, int time, int n_heads,
                               int head_dim);

/* Backward of hl_flash_attention_forward: recomputes P from q, k and lse, then
 *   dV = P^T dO, dP = dO V^T, dS = P*(dP - rowsum(dO*O))*scale, dQ = dS K, dK = dS^T Q
 * with bf16 operands and f32 accumulation (src/tensor/autograd.rs:1626-1914,
 * tensor_core.ptx:3111-4407).  out/dout: bf16 [batch*time, C]; dq, dk, dv: bf16 views with row
 * stride ld_dqkv (may be column slices of one fused gradient buffer).  dK and dV are summed in
 * tensor memory in a fixed order; dQ tiles are summed with f32 reductions whose order is not
 * fixed.  Uses the context's scratch arena (f32 dQ accumulator and row sums). */
int hl_flash_attention_backward(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv,
                                const void* out, long long ld_out, const void* dout, long long ld_dout,
                                const float* lse, void* dq, void* dk, void* dv, long long ld_dqkv, int batch,
                                int time, int n_heads, int head_dim);

/* ---- product-key memory layer ----------------------------------------------------------------
 * Per-row top-k of stored f32 scores: descending score, ties to the lower index
 * (Tensor::topk_indices_dim1, src/tensor.rs:641-702; kernels.ptx:1780).  cols <= 2048. */
int hl_topk_rows_f32(hl_ctx* ctx, const float* scores, int64_t* out, int rows, int cols, int k);
/* Side scores of the product-key lookup: left[t,s] = q[t,:half] . K_L[s], right[t,s] = q[t,half:] . K_R[s]
 * with the reference's f32 dot order (acc = acc + q[j]*k[j], multiply and add rounded separately,
 * src/memory_transformer.rs:2029-2034; kernels.ptx:1873), so that equal inputs give equal score
 * bits and therefore equal indices. */
int hl_product_key_side_scores_f32(hl_ctx* ctx, const float* query, long long ld_query, const float* left_keys,
                                   const float* right_keys, float* left_scores, float* right_scores, int tokens,
                                   int side, int key_dim);
/* Top-`beam` per side (desc score, asc index), beam^2 f32 sums, top_k by (desc sum, asc slot);
 * slot = left*side + right (src/memory_transformer.rs:847-924; kernels.ptx:2121).  beam <= 32. */
int hl_product_key_topk_from_side_scores(hl_ctx* ctx, const float* left_scores, const float* right_scores,
                                         int64_t* out, int tokens, int side, int top_k, int beam);
/* row / side and row % side (src/tensor.rs:1654-1719; kernels.ptx:2263). */
int hl_product_key_split_rows(hl_ctx* ctx, const int64_t* rows, int64_t* left, int64_t* right, long long n, int side);
/* Differentiable re-scoring of the chosen slots.  side > 0: product-key tables
 * (score = q_L . K_L[slot/side] + q_R . K_R[slot%side], src/tensor.rs:3593-3769; kernels.ptx:2317);
 * side == 0: exact lookup over one [slots, key_dim] table (src/tensor.rs:3465-3548; kernels.ptx:3028). */
int hl_memory_selected_scores_forward(hl_ctx* ctx, const int64_t* indices, const float* query, long long ld_query,
                                      const float* left_or_keys, const float* right_keys, float* scores, int tokens,
                                      int top_k, int side, int key_dim, int slots);
/* dq and the key-table gradients (added into zero-initialised or running tables with f32 atomics,
 * repeats accumulate; src/tensor/autograd.rs:2325-2494; kernels.ptx:2417-2624, :3110-3259). */
int hl_memory_selected_scores_backward(hl_ctx* ctx, const int64_t* indices, const float* query, long long ld_query,
                                       const float* left_or_keys, const float* right_keys, const float* grad_scores,
                                       float* grad_query, long long ld_grad_query, float* grad_left_or_keys,
                                       float* grad_right_keys, int tokens, int top_k, int side, int key_dim,
                                       int slots);
/* Row softmax and its gradient (Tensor::softmax_dim(1), src/tensor.rs:4521-4602; kernels.ptx:2625, :2697). */
int hl_softmax_rows_f32(hl_ctx* ctx, const float* x, float* y, int rows, int cols);
int hl_softmax_rows_backward_f32(hl_ctx* ctx, const float* y, const float* grad_y, float* grad_x, int rows, int cols);
/* out[t,:] = sum_k w[t,k] V[idx[t,k],:] and its gradients (dw = dout . V row; dV scatter-add with f32
 * atomics) (src/tensor.rs:3771-3900, src/tensor/autograd.rs:2263-2323; kernels.ptx:2796-3027). */
int hl_memory_weighted_value_forward(hl_ctx* ctx, const int64_t* indices, const float* weights, const float* values,
                                     float* out, int tokens, int top_k, int rows, int dim);
int hl_memory_weighted_value_backward(hl_ctx* ctx, const int64_t* indices, const float* weights, const float* values,
                                      const float* grad_out, float* grad_weights, float* grad_values, int tokens,
                                      int top_k, int rows, int dim);
/* AdamW on the set of selected rows: duplicates update once, an optional byte mask filters rows
 * (AdamW::step_sparse_rows_mut, src/nn.rs:2256-2323, :2899-2939; kernels.ptx:537-811).  row_flags is a
 * caller-owned zeroed byte per row; it is left zeroed.  zero_grad_rows != 0 also clears the gradient
 * rows that were consumed.  The caller advances the step counter and passes the bias corrections. */
/* Row masks and packed rows (reference: cuda_selected_rows_mask, cuda_bool_mask_to_i64_indices,
 * cuda_memory_gather_selected_grad_rows_f32_i64 and its scatter twin, src/tensor.rs:1312-1353, :2245-2337,
 * kernels.ptx:673-811), the pieces of the sparse data-parallel exchange:
 *   hl_mark_rows_u8        flags[r] = 1 for every selected row r (and row_mask[r] != 0 when a mask is given)
 *   hl_mask_to_indices_u8  ascending row numbers of the non-zero bytes, and their count (int on the device)
 *   hl_gather_rows_f32     dst[i,:] = src[indices[i],:]      hl_scatter_rows_f32  dst[indices[i],:] = src[i,:] */
int hl_mark_rows_u8(hl_ctx* ctx, const int64_t* selected_rows, long long n_selected, const unsigned char* row_mask,
                    unsigned char* flags, int rows);
int hl_mask_to_indices_u8(hl_ctx* ctx, const unsigned char* mask, int rows, int64_t* out_indices, int* count_dev);
int hl_gather_rows_f32(hl_ctx* ctx, const float* src, const int64_t* indices, int n, int dim, float* dst);
int hl_scatter_rows_f32(hl_ctx* ctx, const float* src, const int64_t* indices, int n, int dim, float* dst);
/* Adds to *sum_dev (f64 on the device, zeroed by the caller) the sum of squares of the gradient rows in the
 * selected set (same set rule and mask as below): the sparse clip norm is taken over active rows only
 * (AdamW::clip_scale_for_sparse_row_updates, src/nn.rs:2667-2774).  row_flags as below. */
int hl_sparse_rows_sum_squares_f32(hl_ctx* ctx, const float* grad, const int64_t* selected_rows, long long n_selected,
                                   const unsigned char* row_mask, unsigned char* row_flags, int rows, int row_dim,
                                   double* sum_dev);
int hl_sparse_adamw_rows_f32(hl_ctx* ctx, float* param, float* grad, float* m, float* v,
                             const int64_t* selected_rows, long long n_selected, const unsigned char* row_mask,
                             unsigned char* row_flags, int rows, int row_dim, const hl_adamw_params* hp,
                             int zero_grad_rows);

/* ---- NCCL data-parallel plumbing ------------------------------------------------------------
 * Same surface as the reference's NcclUniqueId / NcclCommunicator (cuda.rs:305-349,
 * :8049-8233): a 128-byte unique id made on one rank and handed to the others by the caller,
 * init_rank, in-place f32 sum all-reduce, abort.  NCCL is opened at run time. */
int hl_nccl_version(int* out);
int hl_nccl_unique_id(unsigned char out[128]);
int hl_nccl_init(hl_ctx* ctx, int rank, int world, const unsigned char id[128]);
int hl_nccl_allreduce_f32(hl_ctx* ctx, float* buf_dev, size_t count);
/* Byte-wise maximum over the ranks, in place: the union of per-rank row masks
 * (src/bin/heirloom/runtime.rs:4171-4214). */
int hl_nccl_allreduce_max_u8(hl_ctx* ctx, unsigned char* buf_dev, size_t count);
int hl_nccl_abort(hl_ctx* ctx);
int hl_nccl_destroy(hl_ctx* ctx);

/* Bucket arithmetic of the gradient exchange (host only, no GPU needed): the gradient arena of
 * `arena_elems` f32 values is cut into consecutive buckets of `bucket_elems` (25 MiB = 6,553,600 by
 * default; the last one is shorter).  hl_ddp_ready_buckets lists, from `next_bucket` on, the
 * buckets that lie wholly below `done_elems` (every gradient before that offset is final) and
 * returns how many it wrote (-1 on bad arguments).  The reference reduces one tensor at a time
 * after backward (src/nn.rs:2083-2138); this is the schedule that replaces it. */
long long hl_ddp_bucket_count(long long arena_elems, long long bucket_elems);
int hl_ddp_ready_buckets(long long arena_elems, long long bucket_elems, long long next_bucket, long long done_elems,
                         long long* starts, long long* counts, int capacity);

/* ---- training step of the dense decoder LM --------------------------------------------------
 * The reference's N-layer pre-LayerNorm decoder (MemoryTransformerLm without memory layers,
 * src/memory_transformer.rs:1217-1261): learned positions, separate q/k/v/out projections with
 * biases, GELU MLP, untied lm_head with bias, mean next-token cross-entropy, coupled AdamW.
 * Parameter indices follow named_parameters order (src/memory_transformer.rs:2098-2117);
 * hl_decoder_param_info returns the reference's names, so a state dict moves across unchanged. */
enum { HL_PRECISION_F32 = 0, HL_PRECISION_AMP_BF16 = 1 };
typedef struct {
  int vocab, d_model, n_layers, n_heads, d_ff, context;
  int batch;     /* sequences per step on this rank; tokens per step = batch * context */
  int precision; /* HL_PRECISION_AMP_BF16: AmpBf16Policy::cuda_training (src/amp.rs:24-41) */
} hl_decoder_config;
typedef struct {
  float lr, beta1, beta2, eps, weight_decay;
  float clip_norm; /* <= 0: no clipping (AdamW::new default, src/nn.rs:1941-2005) */
} hl_adamw_config;
typedef struct hl_decoder hl_decoder;

int hl_decoder_create(hl_ctx* ctx, const hl_decoder_config* cfg, hl_decoder** out);
/* The same decoder with product-key memory feed-forward blocks at the listed block indices and
 * one shared table set (MemoryTransformerLm with memory layers, src/memory_transformer.rs:1217-1261,
 * :1101-1125; memory feed-forward :742-781; gated value path = memory_plus).  Extra parameters,
 * in state-dict order after the embeddings: shared_memory.product_key_left/right
 * [sqrt(slots), key_dim/2], shared_memory.value [slots, value_dim]; per memory block
 * feed_forward.memory.{query_proj,gate_proj,out_proj}.  memory_heads must be 1 like the reference
 * (src/memory_transformer.rs:683-688).  The optimizer step is the reference's `Full` policy: dense
 * AdamW over every parameter, tables included (runtime.rs:2416-2453).  Under
 * HL_PRECISION_AMP_BF16 the three projections use bf16 operands on the tensor cores (the
 * reference keeps them f32, :787-789); lookup, scores, softmax, gather and gate stay f32. */
typedef struct {
  int n_memory_layers;
  int memory_layers[16];
  int slots, key_dim, value_dim, top_k;
  int memory_heads;
} hl_memory_config;
int hl_memory_decoder_create(hl_ctx* ctx, const hl_decoder_config* cfg, const hl_memory_config* mem,
                             hl_decoder** out);
/* The reference's `SparseRows` optimizer policy for the memory model (runtime.rs:2424-2435;
 * descriptors memory_sparse_adamw_updates, src/memory_transformer.rs:1293-1424; step
 * AdamW::step_sparse_rows_mut, src/nn.rs:2256-2323): row-set AdamW on product_key_left,
 * product_key_right (rows slot/side and slot%side of every selected slot) and the value table
 * (selected slots), rows chosen by several blocks or tokens updated once; nothing else is
 * updated and the step counter advances by one.  With a clip norm the scale comes from the active
 * rows only; under data parallelism the rows are the union over the ranks.  When SMFT masks are set
 * (below), a row is updated only where its table's mask is non-zero. */
int hl_decoder_optimizer_step_sparse_rows(hl_decoder* model);
/* The optimizer step under one of the reference's memory update policies (`MemoryUpdatePolicy`,
 * src/memory_transformer.rs:26-32; dispatch `step_memory_optimizer`, src/bin/heirloom/runtime.rs:2416-2452):
 *   FULL         dense AdamW on every parameter (= hl_decoder_optimizer_step)
 *   MEMORY_ONLY  dense AdamW on the memory tables alone, clip norm over those tables
 *                (AdamW::step_parameter_indices_mut, src/nn.rs:2222-2254)
 *   SPARSE_ROWS  = hl_decoder_optimizer_step_sparse_rows
 *   FROZEN       nothing is updated and the step counter stays
 * and one policy the reference does not have:
 *   DENSE_PLUS_SPARSE_VALUES  dense AdamW on everything except the value table, row-set AdamW on the
 *                value rows the step selected (SMFT value mask honoured), one step count, one clip
 *                factor over the dense gradients plus the active value rows. */
enum {
  HL_MEMORY_UPDATE_FULL = 0,
  HL_MEMORY_UPDATE_MEMORY_ONLY = 1,
  HL_MEMORY_UPDATE_SPARSE_ROWS = 2,
  HL_MEMORY_UPDATE_FROZEN = 3,
  HL_MEMORY_UPDATE_DENSE_PLUS_SPARSE_VALUES = 4
};
int hl_decoder_optimizer_step_policy(hl_decoder* model, int policy);
/* SMFT (sparse memory fine-tuning) support.
 *   hl_memory_access_count_rows_i64_u64: counts[r] += occurrences of r in selected_rows, 64-bit atomic
 *     adds; counts is caller-owned device memory [slots] (zero it for a fresh histogram); a row outside
 *     [0, slots) sets the bad-index status (memory_access_count_rows_i64_u64,
 *     heirloom-kernels/src/cuda.rs:2052-2088, kernels.ptx:813-886).
 *   hl_decoder_memory_access_counts: adds the selections of the last forward pass of every memory block
 *     (MemoryTransformerLm::memory_access_counts, src/memory_transformer.rs:1561-1583).
 *   hl_decoder_set_smft_masks: byte masks (host memory) over the value rows [slots] and the rows of the
 *     two half-key tables [side] each, used by the sparse-rows step
 *     (memory_sparse_adamw_updates_with_mask, src/memory_transformer.rs:1426-1468); three null
 *     pointers switch masking off. */
int hl_memory_access_count_rows_i64_u64(hl_ctx* ctx, const int64_t* selected_rows, long long n_selected, int slots,
                                        unsigned long long* counts);
int hl_decoder_memory_access_counts(hl_decoder* model, unsigned long long* counts_dev);
int hl_decoder_set_smft_masks(hl_decoder* model, const unsigned char* value_mask_host,
                              const unsigned char* left_mask_host, const unsigned char* right_mask_host);
/* Slots chosen by the last forward of one memory block: int64 [batch*context, top_k]. */
int hl_decoder_selected_indices(hl_decoder* model, int layer, int64_t* host, long long count);
void hl_decoder_destroy(hl_decoder* model);
int hl_decoder_param_count(hl_decoder* model);
int hl_decoder_param_info(hl_decoder* model, int index, char* name_out, size_t name_cap, long long* numel,
                          int* rank, long long shape_out[2]);
/* Host <-> device copies of one parameter / its gradient / its AdamW moments (f32, C order). */
int hl_decoder_set_param(hl_decoder* model, int index, const float* host, long long numel);
int hl_decoder_get_param(hl_decoder* model, int index, float* host, long long numel);
int hl_decoder_get_grad(hl_decoder* model, int index, float* host, long long numel);
int hl_decoder_get_moments(hl_decoder* model, int index, float* m_host, float* v_host, long long numel);
/* AdamW::new + with_* (src/nn.rs:1941-2005): resets the step counter and the moments. */
int hl_decoder_set_optimizer(hl_decoder* model, const hl_adamw_config* opt);
long long hl_decoder_optimizer_steps(hl_decoder* model);
/* AdamW::load_state (src/nn.rs:2059-2080): moments of one parameter and the step counter, as a
 * checkpoint holds them (optimizer.json written by src/checkpoint.rs:124-146). */
int hl_decoder_set_moments(hl_decoder* model, int index, const float* m_host, const float* v_host, long long numel);
int hl_decoder_set_optimizer_steps(hl_decoder* model, long long steps);
/* Forward only, no gradients (the loss inside evaluate_token_loss, src/memory_transformer.rs:1813-1912):
 * mean cross-entropy over `sequences` (1..batch) rows of `context` tokens; the value is copied to the host. */
int hl_decoder_eval_loss(hl_decoder* model, const int64_t* tokens_dev, const int64_t* targets_dev, int sequences,
                         float* loss_host);
/* next_token_logits (src/memory_transformer.rs:1930-1984): one window of 1..context tokens, full-window
 * forward, the `vocab` logits of its last position copied to the host. */
int hl_decoder_next_token_logits(hl_decoder* model, const int64_t* window_dev, int window_len, float* logits_host);
/* zero_grad + loss + backward (src/bin/heirloom/commands/training.rs:125-167) on device-resident
 * i64 tokens/targets of shape [batch, context].  With an NCCL communicator on the context,
 * 25 MiB gradient buckets are all-reduced on the collective stream as backward produces them. */
int hl_decoder_forward_backward(hl_decoder* model, const int64_t* tokens_dev, const int64_t* targets_dev);
/* AdamW::step_mut (src/nn.rs:2156-2220); with world > 1 the summed gradients are scaled by
 * 1/world inside the update (src/nn.rs:2100-2117). */
int hl_decoder_optimizer_step(hl_decoder* model);
/* forward_backward + optimizer_step, nothing leaves the device. */
int hl_decoder_train_step_device(hl_decoder* model, const int64_t* tokens_dev, const int64_t* targets_dev);
/* The whole step from host memory: copies tokens/targets in, runs the step, copies the loss out
 * and waits for it (the reference reads the loss every step too, reports.rs:285-308). */
int hl_decoder_train_step(hl_decoder* model, const int64_t* tokens_host, const int64_t* targets_host,
                          float* loss_host);
/* Loss of the last forward (waits for the compute stream). */
int hl_decoder_loss(hl_decoder* model, float* loss_host);
/* Kernels launched by the last forward_backward + optimizer_step. */
unsigned long long hl_decoder_launches_last_step(hl_decoder* model);
/* Data parallelism: how long the compute stream sat idle in its waits for the collective stream since the last call
 * (sum over the waits, and their number), measured with timing events while hl_profile_enable is on; 0 otherwise.
 * Synchronises the compute stream.  The reference times its exchange the same way, as the all-reduce's own event
 * timer (NcclCommunicator::start_event_timer, heirloom-kernels/src/cuda.rs:8049-8233). */
int hl_decoder_comm_exposed_ms(hl_decoder* model, float* total_ms, int* waits);

#ifdef __cplusplus
}
#endif
#endif /* HEIRLOOM_B200_H */
