// Training-step executor for the dense pre-LayerNorm decoder LM: forward, backward, bucketed
// gradient all-reduce overlapped with backward, and the fused AdamW update, on preplanned
// arenas.  It reproduces the reference's AMP-bf16 dataflow
//   MemoryTransformerLm::forward_amp_bf16 / loss_amp_bf16 (src/memory_transformer.rs:1636-1670),
//   block (src/memory_transformer.rs:1153-1172), attention (src/nn.rs:718-788),
//   feed-forward (src/nn.rs:873-884), Linear (src/nn.rs:338-450),
//   backward operand rounding (src/tensor/autograd.rs:593-851),
//   AdamW::step_mut (src/nn.rs:2156-2220) and the data-parallel exchange
//   AdamW::all_reduce_cuda_gradients_nccl (src/nn.rs:2083-2138)
// with every bf16 round trip of that path realised as "store the activation in bf16".
//
// Parameters live in one flat f32 arena (plus f32 gradients, AdamW moments and a bf16 shadow
// used as GEMM operands), ordered by the time their gradient becomes final in backward
// (lm_head first, embeddings last) so that fixed-size buckets of the gradient arena can be
// all-reduced on the collective stream while backward is still running.
#include <cstring>
#include <string>
#include <vector>

#include "kernels.h"

namespace hl {
namespace {

constexpr size_t kAlignElems = 64;
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct Slot {
  std::string name;
  size_t offset, numel;
  int rank;
  long long shape[2];
};

struct LayerOffsets {
  size_t w2, b2, w1, b1, ln2g, ln2b, wo, bo, wqkv, bqkv, ln1g, ln1b;
  // memory feed-forward blocks use these instead of w1/b1/w2/b2
  bool is_memory = false;
  size_t wq_m = 0, bq_m = 0, wg_m = 0, bg_m = 0, wout_m = 0, bout_m = 0;
  // bias of the projection that writes the block output (fc2 or the memory out_proj)
  size_t out_bias() const { return is_memory ? bout_m : b2; }
};

// Per memory layer: everything the backward needs (all f32, as in the reference the memory
// feed-forward runs in f32 also under AMP, src/memory_transformer.rs:787-789).
struct MemoryActs {
  float *query = nullptr, *weights = nullptr, *weighted = nullptr, *gpre = nullptr, *gate = nullptr, *mv = nullptr;
  int64_t* idx = nullptr;
  __nv_bfloat16* mv_b = nullptr;  // amp route: [N, 2*value_dim] = [hi | lo] pieces of mv
  // amp route: the three projection weights as bf16 pieces along the contraction (hl_split_bf16_f32),
  // rebuilt from the f32 parameters at the start of every forward pass
  __nv_bfloat16 *wq3 = nullptr, *wg3 = nullptr, *wout3 = nullptr;
};

struct LayerActs {
  __nv_bfloat16 *a, *qkv, *o, *r, *c, *h, *g;
  float *lse, *mean1, *rstd1, *mean2, *rstd2;
};

}  // namespace
}  // namespace hl

using namespace hl;

struct hl_decoder {
  hl_ctx* ctx = nullptr;
  hl_decoder_config cfg{};
  int N = 0;
  // parameter arenas
  size_t arena = 0;
  float *params = nullptr, *grads = nullptr, *m = nullptr, *v = nullptr;
  __nv_bfloat16* shadow = nullptr;
  std::vector<Slot> slots;  // state-dict order
  size_t off_head_w = 0, off_head_b = 0, off_lnf_g = 0, off_lnf_b = 0, off_pos = 0, off_tok = 0;
  std::vector<LayerOffsets> lo;
  // activations
  uint8_t* act_arena = nullptr;
  size_t act_bytes = 0;
  std::vector<__nv_bfloat16*> x;  // x[l] is the input of block l; x[L] the final residual stream
  std::vector<LayerActs> la;
  __nv_bfloat16 *z = nullptr, *dlogits = nullptr, *dxb = nullptr, *dh = nullptr, *dob = nullptr, *dqkv = nullptr;
  // head sizes other than 64 and 128 on the bf16 route: attention runs through the f32 kernels on these shared buffers
  bool flash_ok = true;
  float *fa_q = nullptr, *fa_k = nullptr, *fa_v = nullptr, *fa_o = nullptr, *fa_probs = nullptr, *fa_dq = nullptr,
        *fa_dk = nullptr, *fa_dv = nullptr, *fa_do = nullptr;
  float *logits = nullptr, *meanf = nullptr, *rstdf = nullptr, *dx0 = nullptr, *dx1 = nullptr, *dtmp = nullptr;
  int64_t *tokens = nullptr, *targets = nullptr;
  FoldBatch fold;  // column reductions of one block's backward, folded by one launch before its buckets are flushed
  float* loss_dev = nullptr;
  float* loss_host = nullptr;  // pinned
  float* norm_dev = nullptr;
  double* norm_dev64 = nullptr;  // f64 sum of squares over active sparse rows
  float* norm_host = nullptr;  // pinned
  // optimizer
  bool has_opt = false;
  hl_adamw_config opt{};
  long long step = 0;
  AdamPlan* plan = nullptr;
  // data-parallel buckets over the gradient arena
  size_t bucket_elems = 6553600;  // 25 MiB of f32
  size_t next_bucket = 0, n_buckets = 0;
  std::vector<cudaEvent_t> bucket_ready;
  std::vector<cudaEvent_t> bucket_done;  // recorded on the collective stream after each bucket's all-reduce
  bool comm_pending = false;             // the compute stream has not yet waited for this step's collectives
  cudaEvent_t comm_done = nullptr;
  // row-union exchanges: which rows the ranks touched is known long before their gradients are (the token ids when the
  // step starts, the selected slots when forward ends), so the union and its size are formed then, on the collective
  // stream, and the host finds the size ready when it queues the exchange itself at the end of backward
  cudaEvent_t rows_known = nullptr, tok_count_ready = nullptr, val_count_ready = nullptr;
  bool tok_prepared = false, val_prepared = false;
  // while per-kernel timing is on: events around every wait of the compute stream for the collective stream, so that
  // the time the step spends exposed to the gradient exchange can be read back (hl_decoder_comm_exposed_ms)
  std::vector<cudaEvent_t> wait_begin, wait_end;
  size_t waits_recorded = 0;
  unsigned long long launches_last_step = 0;
  // product-key memory (shared tables, MemoryTransformerLm with memory layers)
  bool has_memory = false;
  hl_memory_config mem{};
  int side = 0;
  size_t off_kl = 0, off_kr = 0, off_val = 0;
  size_t tables_end = 0;  // first arena element after the value table
  AdamPlan *plan_tables = nullptr, *plan_no_values = nullptr;  // the memory tables alone; everything but the value table
  std::vector<MemoryActs> ma;  // indexed by layer; empty entries for dense layers
  float *m_ls = nullptr, *m_rs = nullptr, *m_scores = nullptr, *m_dmv = nullptr, *m_dweighted = nullptr, *m_dgate = nullptr,
        *m_dgpre = nullptr, *m_dw = nullptr, *m_dscores = nullptr, *m_dq = nullptr, *m_dc2 = nullptr;
  __nv_bfloat16 *m_dgpre_b = nullptr, *m_dq_b = nullptr;
  // amp route, backward of the three memory projections at f32 accuracy: bf16 pieces of the f32 operands, side by
  // side along the columns where the contraction runs along a row, one below the other where it runs down the rows
  __nv_bfloat16 *p_dx_side = nullptr, *p_dx_rows = nullptr, *p_mv_rows = nullptr, *p_dg_side = nullptr, *p_dg_rows = nullptr,
                *p_dq_side = nullptr, *p_dq_rows = nullptr, *p_wout_rows = nullptr, *p_wg_rows = nullptr, *p_wq_rows = nullptr;
  unsigned char* m_row_flags = nullptr;
  unsigned char *smft_value_mask = nullptr, *smft_left_mask = nullptr, *smft_right_mask = nullptr;  // [slots], [side], [side]
  bool smft_on = false;  // the sparse-rows step filters its rows through the three masks
  float* m_packed = nullptr;         // gradient rows of the union, packed for the all-reduce (own allocation)
  size_t packed_rows_cap = 0;        // rows it holds
  // data-parallel exchange of the token-embedding gradient as the union of the rows any rank's batch touched
  bool sparse_tok_exchange = true;
  unsigned char* tok_flags = nullptr;  // [vocab]
  int64_t* tok_union_rows = nullptr;   // [vocab]
  int* tok_union_count = nullptr;
  int* tok_union_count_host = nullptr;  // pinned
  float* tok_packed = nullptr;
  size_t tok_packed_cap = 0;
  int64_t* m_union_rows = nullptr;   // rows of the value table selected by any rank this step
  int* m_union_count = nullptr;      // device count of them
  int* m_union_count_host = nullptr; // pinned mirror
  int union_n = -1;                  // rows in the union after the last exchange, -1 before any
  int64_t *m_sel_all = nullptr, *m_sel_left = nullptr, *m_sel_right = nullptr;  // concatenated selections of all memory blocks
  // f32 route (reference f32 semantics: f32 tensors, f64 accumulation inside every op)
  struct F32Layer {
    float *a, *q, *k, *v, *probs, *o, *pr, *r, *c, *h, *g, *f;
  };
  std::vector<float*> xf;  // residual stream per block input, f32
  std::vector<F32Layer> lf;
  float *zf = nullptr, *tmp_f = nullptr, *tmp2_f = nullptr, *dlogits_f = nullptr, *d_a = nullptr, *d_b = nullptr,
        *d_c = nullptr, *d_q = nullptr, *d_k = nullptr, *d_v = nullptr, *d_wide = nullptr, *d_wide2 = nullptr;
};

namespace hl {
namespace {

// Lays the parameters out in gradient-completion order and records the name -> slice map in
// the reference's state-dict order (src/memory_transformer.rs:2098-2117).
void plan_parameters(hl_decoder* m) {
  const hl_decoder_config& c = m->cfg;
  const long long d = c.d_model, F = c.d_ff, V = c.vocab, T = c.context;
  size_t cur = 0;
  std::vector<Slot> tmp;
  auto add = [&](const std::string& name, size_t numel, int rank, long long s0, long long s1) {
    const size_t off = cur;
    cur = align_up(cur + numel, kAlignElems);
    tmp.push_back(Slot{name, off, numel, rank, {s0, s1}});
    return off;
  };
  m->off_head_w = add("lm_head.weight", (size_t)V * d, 2, V, d);
  m->off_head_b = add("lm_head.bias", (size_t)V, 1, V, 0);
  m->off_lnf_g = add("ln_f.weight", (size_t)d, 1, d, 0);
  m->off_lnf_b = add("ln_f.bias", (size_t)d, 1, d, 0);
  m->lo.resize(c.n_layers);
  for (int l = c.n_layers - 1; l >= 0; --l) {
    const std::string b = "block." + std::to_string(l) + ".";
    LayerOffsets& o = m->lo[l];
    o.is_memory = false;
    for (int i = 0; m->has_memory && i < m->mem.n_memory_layers; ++i) o.is_memory |= m->mem.memory_layers[i] == l;
    if (o.is_memory) {
      const long long kd = m->mem.key_dim, vd = m->mem.value_dim;
      const std::string f = b + "feed_forward.memory.";
      o.wout_m = add(f + "out_proj.weight", (size_t)d * vd, 2, d, vd);
      o.bout_m = add(f + "out_proj.bias", (size_t)d, 1, d, 0);
      o.wg_m = add(f + "gate_proj.weight", (size_t)vd * d, 2, vd, d);
      o.bg_m = add(f + "gate_proj.bias", (size_t)vd, 1, vd, 0);
      o.wq_m = add(f + "query_proj.weight", (size_t)kd * d, 2, kd, d);
      o.bq_m = add(f + "query_proj.bias", (size_t)kd, 1, kd, 0);
      o.w2 = o.b2 = o.w1 = o.b1 = 0;
    } else {
    o.w2 = add(b + "feed_forward.dense.fc2.weight", (size_t)d * F, 2, d, F);
    o.b2 = add(b + "feed_forward.dense.fc2.bias", (size_t)d, 1, d, 0);
    o.w1 = add(b + "feed_forward.dense.fc1.weight", (size_t)F * d, 2, F, d);
    o.b1 = add(b + "feed_forward.dense.fc1.bias", (size_t)F, 1, F, 0);
    }
    o.ln2g = add(b + "ln2.weight", (size_t)d, 1, d, 0);
    o.ln2b = add(b + "ln2.bias", (size_t)d, 1, d, 0);
    o.wo = add(b + "attention.out_proj.weight", (size_t)d * d, 2, d, d);
    o.bo = add(b + "attention.out_proj.bias", (size_t)d, 1, d, 0);
    // q, k, v are three reference Linears stored back to back so one [3d, d] GEMM serves them
    o.wqkv = cur;
    add(b + "attention.q_proj.weight", (size_t)d * d, 2, d, d);
    cur = o.wqkv + (size_t)d * d;
    add(b + "attention.k_proj.weight", (size_t)d * d, 2, d, d);
    cur = o.wqkv + 2 * (size_t)d * d;
    add(b + "attention.v_proj.weight", (size_t)d * d, 2, d, d);
    o.bqkv = cur;
    add(b + "attention.q_proj.bias", (size_t)d, 1, d, 0);
    cur = o.bqkv + d;
    add(b + "attention.k_proj.bias", (size_t)d, 1, d, 0);
    cur = o.bqkv + 2 * d;
    add(b + "attention.v_proj.bias", (size_t)d, 1, d, 0);
    o.ln1g = add(b + "ln1.weight", (size_t)d, 1, d, 0);
    o.ln1b = add(b + "ln1.bias", (size_t)d, 1, d, 0);
  }
  if (m->has_memory) {
    const long long half = m->mem.key_dim / 2;
    m->off_kl = add("shared_memory.product_key_left", (size_t)m->side * half, 2, m->side, half);
    m->off_kr = add("shared_memory.product_key_right", (size_t)m->side * half, 2, m->side, half);
    m->off_val = add("shared_memory.value", (size_t)m->mem.slots * m->mem.value_dim, 2, m->mem.slots, m->mem.value_dim);
    m->tables_end = cur;
  }
  m->off_pos = add("position_embedding.weight", (size_t)T * d, 2, T, d);
  m->off_tok = add("token_embedding.weight", (size_t)V * d, 2, V, d);
  m->arena = cur;
  // state-dict order
  auto find = [&](const std::string& n) -> Slot {
    for (const Slot& s : tmp) if (s.name == n) return s;
    return Slot{};
  };
  m->slots.push_back(find("token_embedding.weight"));
  m->slots.push_back(find("position_embedding.weight"));
  if (m->has_memory)
    for (const char* n : {"shared_memory.product_key_left", "shared_memory.product_key_right", "shared_memory.value"})
      m->slots.push_back(find(n));
  for (int l = 0; l < c.n_layers; ++l) {
    const std::string b = "block." + std::to_string(l) + ".";
    for (const char* n : {"ln1.weight", "ln1.bias", "attention.q_proj.weight", "attention.q_proj.bias",
                          "attention.k_proj.weight", "attention.k_proj.bias", "attention.v_proj.weight",
                          "attention.v_proj.bias", "attention.out_proj.weight", "attention.out_proj.bias", "ln2.weight",
                          "ln2.bias"})
      m->slots.push_back(find(b + n));
    if (m->lo[l].is_memory) {
      for (const char* n : {"feed_forward.memory.query_proj.weight", "feed_forward.memory.query_proj.bias",
                            "feed_forward.memory.gate_proj.weight", "feed_forward.memory.gate_proj.bias",
                            "feed_forward.memory.out_proj.weight", "feed_forward.memory.out_proj.bias"})
        m->slots.push_back(find(b + n));
    } else {
      for (const char* n : {"feed_forward.dense.fc1.weight", "feed_forward.dense.fc1.bias", "feed_forward.dense.fc2.weight",
                            "feed_forward.dense.fc2.bias"})
        m->slots.push_back(find(b + n));
    }
  }
  for (const char* n : {"ln_f.weight", "ln_f.bias", "lm_head.weight", "lm_head.bias"}) m->slots.push_back(find(n));
}

template <typename T>
T* carve(uint8_t*& cursor, size_t count) {
  T* p = reinterpret_cast<T*>(cursor);
  cursor += align_up(count * sizeof(T), 256);
  return p;
}

// Buffers of the memory feed-forward blocks; appended to either route's arena.
void plan_memory_buffers(hl_decoder* m, uint8_t*& cur) {
  m->tok_flags = carve<unsigned char>(cur, (size_t)m->cfg.vocab);
  m->tok_union_rows = carve<int64_t>(cur, (size_t)m->cfg.vocab);
  m->tok_union_count = carve<int>(cur, 4);
  if (!m->has_memory) return;
  const size_t N = (size_t)m->N, kd = m->mem.key_dim, vd = m->mem.value_dim, k = m->mem.top_k, d = m->cfg.d_model;
  m->ma.assign(m->cfg.n_layers, MemoryActs{});
  for (int l = 0; l < m->cfg.n_layers; ++l) {
    if (!m->lo[l].is_memory) continue;
    MemoryActs& a = m->ma[l];
    a.query = carve<float>(cur, N * kd);
    a.weights = carve<float>(cur, N * k);
    a.weighted = carve<float>(cur, N * vd);
    a.gpre = carve<float>(cur, N * vd);
    a.gate = carve<float>(cur, N * vd);
    a.mv = carve<float>(cur, N * vd);
    a.idx = carve<int64_t>(cur, N * k);
    a.mv_b = carve<__nv_bfloat16>(cur, N * 2 * vd);
    a.wq3 = carve<__nv_bfloat16>(cur, kd * 3 * d);
    a.wg3 = carve<__nv_bfloat16>(cur, vd * 3 * d);
    a.wout3 = carve<__nv_bfloat16>(cur, d * 3 * vd);
  }
  m->m_ls = carve<float>(cur, N * m->side);
  m->m_rs = carve<float>(cur, N * m->side);
  m->m_scores = carve<float>(cur, N * k);
  m->m_dmv = carve<float>(cur, N * vd);
  m->m_dweighted = carve<float>(cur, N * vd);
  m->m_dgate = carve<float>(cur, N * vd);
  m->m_dgpre = carve<float>(cur, N * vd);
  m->m_dw = carve<float>(cur, N * k);
  m->m_dscores = carve<float>(cur, N * k);
  m->m_dq = carve<float>(cur, N * kd);
  m->m_dc2 = carve<float>(cur, N * d);
  m->m_dgpre_b = carve<__nv_bfloat16>(cur, N * vd);
  m->m_dq_b = carve<__nv_bfloat16>(cur, N * kd);
  if (m->cfg.precision == HL_PRECISION_AMP_BF16) {
    m->p_dx_side = carve<__nv_bfloat16>(cur, N * 2 * d);
    m->p_dx_rows = carve<__nv_bfloat16>(cur, 2 * N * d);
    m->p_mv_rows = carve<__nv_bfloat16>(cur, 3 * N * vd);
    m->p_dg_side = carve<__nv_bfloat16>(cur, N * 2 * vd);
    m->p_dg_rows = carve<__nv_bfloat16>(cur, 3 * N * vd);
    m->p_dq_side = carve<__nv_bfloat16>(cur, N * 2 * kd);
    m->p_dq_rows = carve<__nv_bfloat16>(cur, 3 * N * kd);
    m->p_wout_rows = carve<__nv_bfloat16>(cur, 3 * d * vd);
    m->p_wg_rows = carve<__nv_bfloat16>(cur, 3 * vd * d);
    m->p_wq_rows = carve<__nv_bfloat16>(cur, 3 * kd * d);
  }
  m->m_row_flags = carve<unsigned char>(cur, (size_t)m->mem.slots);
  m->smft_value_mask = carve<unsigned char>(cur, (size_t)m->mem.slots);
  m->smft_left_mask = carve<unsigned char>(cur, (size_t)m->side);
  m->smft_right_mask = carve<unsigned char>(cur, (size_t)m->side);
  m->m_union_rows = carve<int64_t>(cur, (size_t)m->mem.slots);
  m->m_union_count = carve<int>(cur, 4);
  // room for this rank's selections of every memory block, or for the union of all ranks' (at most every slot)
  const size_t all = std::max(N * k * (size_t)m->mem.n_memory_layers, (size_t)m->mem.slots);
  m->m_sel_all = carve<int64_t>(cur, all);
  m->m_sel_left = carve<int64_t>(cur, all);
  m->m_sel_right = carve<int64_t>(cur, all);
}

int plan_activations(hl_decoder* m, bool measure_only, size_t* bytes_out) {
  const hl_decoder_config& c = m->cfg;
  const size_t N = (size_t)m->N, d = c.d_model, F = c.d_ff, V = c.vocab, L = c.n_layers;
  uint8_t* cur = measure_only ? nullptr : m->act_arena;
  uint8_t* base = cur;
  m->x.resize(L + 1);
  m->la.resize(L);
  for (size_t l = 0; l <= L; ++l) m->x[l] = carve<__nv_bfloat16>(cur, N * d);
  for (size_t l = 0; l < L; ++l) {
    LayerActs& a = m->la[l];
    a.a = carve<__nv_bfloat16>(cur, N * d);
    a.qkv = carve<__nv_bfloat16>(cur, N * 3 * d);
    a.o = carve<__nv_bfloat16>(cur, N * d);
    a.r = carve<__nv_bfloat16>(cur, N * d);
    a.c = carve<__nv_bfloat16>(cur, N * d);
    a.h = carve<__nv_bfloat16>(cur, N * F);
    a.g = carve<__nv_bfloat16>(cur, N * F);
    a.lse = carve<float>(cur, N * c.n_heads);
    a.mean1 = carve<float>(cur, N);
    a.rstd1 = carve<float>(cur, N);
    a.mean2 = carve<float>(cur, N);
    a.rstd2 = carve<float>(cur, N);
  }
  m->z = carve<__nv_bfloat16>(cur, N * d);
  m->meanf = carve<float>(cur, N);
  m->rstdf = carve<float>(cur, N);
  m->logits = carve<float>(cur, N * V);
  m->dlogits = carve<__nv_bfloat16>(cur, N * V);
  m->dx0 = carve<float>(cur, N * d);
  m->dx1 = carve<float>(cur, N * d);
  m->dtmp = carve<float>(cur, N * d);
  m->dxb = carve<__nv_bfloat16>(cur, N * d);
  m->dh = carve<__nv_bfloat16>(cur, N * F);
  m->dob = carve<__nv_bfloat16>(cur, N * d);
  m->dqkv = carve<__nv_bfloat16>(cur, N * 3 * d);
  if (!m->flash_ok) {
    m->fa_q = carve<float>(cur, N * d); m->fa_k = carve<float>(cur, N * d); m->fa_v = carve<float>(cur, N * d);
    m->fa_o = carve<float>(cur, N * d); m->fa_do = carve<float>(cur, N * d);
    m->fa_dq = carve<float>(cur, N * d); m->fa_dk = carve<float>(cur, N * d); m->fa_dv = carve<float>(cur, N * d);
    m->fa_probs = carve<float>(cur, (size_t)c.batch * c.n_heads * c.context * c.context);
  }
  plan_memory_buffers(m, cur);
  {
    // partial rows of the column reductions: two layer norms (at most 2 CTAs per SM, three sums each) and the bias
    // column sums (at most 64 slabs) of one block, or the head's
    const size_t sm = (size_t)m->ctx->sm_count;
    const size_t ln = 2 * sm * 3 * d + 64;
    const size_t wide = m->has_memory ? std::max(F, (size_t)(m->mem.key_dim + m->mem.value_dim)) : F;
    const size_t layer = 2 * ln + 64 * (wide + 3 * d) + 4 * 64;
    const size_t head = ln + 64 * V + 2 * 64;
    m->fold.capacity = std::max(layer, head);
    m->fold.scratch = carve<float>(cur, m->fold.capacity);
    m->fold.n = 0;
    m->fold.used = 0;
  }
  m->tokens = carve<int64_t>(cur, N);
  m->targets = carve<int64_t>(cur, N);
  m->loss_dev = carve<float>(cur, 4);
  m->norm_dev = carve<float>(cur, 4);
  m->norm_dev64 = carve<double>(cur, 2);
  *bytes_out = (size_t)(cur - base);
  return HL_OK;
}

int plan_activations_f32(hl_decoder* m, bool measure_only, size_t* bytes_out) {
  const hl_decoder_config& c = m->cfg;
  const size_t N = (size_t)m->N, d = c.d_model, F = c.d_ff, V = c.vocab, L = c.n_layers;
  const size_t BHTT = (size_t)c.batch * c.n_heads * c.context * c.context;
  uint8_t* cur = measure_only ? nullptr : m->act_arena;
  uint8_t* base = cur;
  m->xf.resize(L + 1);
  m->lf.resize(L);
  for (size_t l = 0; l <= L; ++l) m->xf[l] = carve<float>(cur, N * d);
  for (size_t l = 0; l < L; ++l) {
    hl_decoder::F32Layer& a = m->lf[l];
    a.a = carve<float>(cur, N * d);
    a.q = carve<float>(cur, N * d);
    a.k = carve<float>(cur, N * d);
    a.v = carve<float>(cur, N * d);
    a.probs = carve<float>(cur, BHTT);
    a.o = carve<float>(cur, N * d);
    a.pr = carve<float>(cur, N * d);
    a.r = carve<float>(cur, N * d);
    a.c = carve<float>(cur, N * d);
    a.h = carve<float>(cur, N * F);
    a.g = carve<float>(cur, N * F);
    a.f = carve<float>(cur, N * d);
  }
  m->zf = carve<float>(cur, N * d);
  m->logits = carve<float>(cur, N * V);
  m->dlogits_f = carve<float>(cur, N * V);
  m->tmp_f = carve<float>(cur, N * std::max(std::max(std::max(d, F), V),
                                            m->has_memory ? (size_t)std::max(m->mem.key_dim, m->mem.value_dim) : (size_t)1));
  m->tmp2_f = carve<float>(cur, N * d);
  m->d_a = carve<float>(cur, N * d);
  m->d_b = carve<float>(cur, N * d);
  m->d_c = carve<float>(cur, N * d);
  m->d_q = carve<float>(cur, N * d);
  m->d_k = carve<float>(cur, N * d);
  m->d_v = carve<float>(cur, N * d);
  m->d_wide = carve<float>(cur, N * F);
  m->d_wide2 = carve<float>(cur, N * F);
  plan_memory_buffers(m, cur);
  m->tokens = carve<int64_t>(cur, N);
  m->targets = carve<int64_t>(cur, N);
  m->loss_dev = carve<float>(cur, 4);
  m->norm_dev = carve<float>(cur, 4);
  m->norm_dev64 = carve<double>(cur, 2);
  *bytes_out = (size_t)(cur - base);
  return HL_OK;
}

struct Gemm {
  hl_decoder* m;
  int run(int M, int N, int K, const void* a, long long lda, int al, const void* b, long long ldb, int bl, void* c,
          long long ldc, int out_dtype, int epi = HL_EPI_NONE, const float* bias = nullptr, const void* aux_in = nullptr,
          long long ld_aux_in = 0, void* aux_out = nullptr, long long ld_aux_out = 0, int a_k_period = 0,
          int b_k_period = 0) const {
    hl_gemm_desc d{};
    d.m = M; d.n = N; d.k = K;
    d.a_k_period = a_k_period;
    d.b_k_period = b_k_period;
    d.a_layout = al; d.b_layout = bl;
    d.lda = lda; d.ldb = ldb; d.ldc = ldc;
    d.epilogue = epi; d.out_dtype = out_dtype; d.split_k = 0;
    d.ld_aux_in = ld_aux_in; d.ld_aux_out = ld_aux_out;
    return gemm_bf16_ctx(m->ctx, &d, a, b, c, bias, aux_in, aux_out);
  }
};

#define HL_TRY(expr)            \
  do {                          \
    int _rc = (expr);           \
    if (_rc != HL_OK) return _rc; \
  } while (0)

// ---- memory feed-forward core (both routes): lookup, re-scoring, softmax, weighted value -----------
// query [N, key_dim] f32 is already in ma[l].query (MemoryFeedForward::forward_named,
// src/memory_transformer.rs:742-781).
int memory_core_forward(hl_decoder* m, int l) {
  hl_ctx* ctx = m->ctx;
  MemoryActs& a = m->ma[l];
  const float* P = m->params;
  const int N = m->N, kd = m->mem.key_dim, vd = m->mem.value_dim, k = m->mem.top_k, side = m->side;
  const int beam = std::min(side, std::max(k, (int)ceil(sqrt((double)k))));  // product_key_beam, :2014-2016
  // timed as one family ("other" in the per-kernel profile); work = table rows gathered, in bytes
  ProfileScope prof(ctx, HL_PROF_OTHER, (double)N * k * (double)(kd + vd) * 4.0 + 2.0 * (double)N * side * 4.0);
  HL_TRY(hl_product_key_side_scores_f32(ctx, a.query, kd, P + m->off_kl, P + m->off_kr, m->m_ls, m->m_rs, N, side, kd));
  HL_TRY(hl_product_key_topk_from_side_scores(ctx, m->m_ls, m->m_rs, a.idx, N, side, k, beam));
  HL_TRY(hl_memory_selected_scores_forward(ctx, a.idx, a.query, kd, P + m->off_kl, P + m->off_kr, m->m_scores, N, k, side, kd,
                                           m->mem.slots));
  HL_TRY(hl_softmax_rows_f32(ctx, m->m_scores, a.weights, N, k));
  return hl_memory_weighted_value_forward(ctx, a.idx, a.weights, P + m->off_val, a.weighted, N, k, m->mem.slots, vd);
}

// dweighted -> m_dq (gradient of the query) and the table gradients (added into the arena).
int memory_core_backward(hl_decoder* m, int l, const float* dweighted) {
  hl_ctx* ctx = m->ctx;
  MemoryActs& a = m->ma[l];
  const float* P = m->params;
  float* G = m->grads;
  const int N = m->N, kd = m->mem.key_dim, vd = m->mem.value_dim, k = m->mem.top_k, side = m->side;
  ProfileScope prof(ctx, HL_PROF_OTHER, (double)N * k * (double)(kd + 3 * vd) * 4.0);
  HL_TRY(hl_memory_weighted_value_backward(ctx, a.idx, a.weights, P + m->off_val, dweighted, m->m_dw, G + m->off_val, N, k,
                                           m->mem.slots, vd));
  HL_TRY(hl_softmax_rows_backward_f32(ctx, a.weights, m->m_dw, m->m_dscores, N, k));
  return hl_memory_selected_scores_backward(ctx, a.idx, a.query, kd, P + m->off_kl, P + m->off_kr, m->m_dscores, m->m_dq, kd,
                                            G + m->off_kl, G + m->off_kr, N, k, side, kd, m->mem.slots);
}

// Table gradients are sums over scattered rows: they start every backward at zero.
int zero_memory_table_grads(hl_decoder* m) {
  if (!m->has_memory) return HL_OK;
  const size_t count = m->off_val + (size_t)m->mem.slots * m->mem.value_dim - m->off_kl;
  HL_CUDA(cudaMemsetAsync(m->grads + m->off_kl, 0, sizeof(float) * count, m->ctx->stream));
  return HL_OK;
}

// ---- attention for head sizes the tcgen05 kernels are not built for (they take head_dim 64 and 128) -------------
// The bf16 q, k, v are widened to f32 (exact), the f32 attention kernels run on them and their results are rounded to
// bf16 where the flash route stores bf16 (attention output, dQ/dK/dV).  Probabilities are not kept per layer: the
// backward pass runs the forward kernel again into the shared probability buffer.
__global__ void rows_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src, float* __restrict__ dst,
                                        long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[(i / cols) * ld_src + (i % cols)]);
}
__global__ void rows_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long ld_dst,
                                        long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[(i / cols) * ld_dst + (i % cols)] = __float2bfloat16_rn(src[i]);
}

int widen_rows(hl_ctx* ctx, const __nv_bfloat16* src, long long ld_src, float* dst, long long rows, int cols) {
  const long long want = ceil_div_ll(rows * cols, 256);
  rows_bf16_to_f32_kernel<<<(unsigned)std::min<long long>(want, (long long)ctx->sm_count * 16), 256, 0, ctx->stream>>>(
      src, ld_src, dst, rows, cols);
  HL_LAUNCH_CHECK("rows_bf16_to_f32_kernel");
  count_launch(ctx);
  return HL_OK;
}
int narrow_rows(hl_ctx* ctx, const float* src, __nv_bfloat16* dst, long long ld_dst, long long rows, int cols) {
  const long long want = ceil_div_ll(rows * cols, 256);
  rows_f32_to_bf16_kernel<<<(unsigned)std::min<long long>(want, (long long)ctx->sm_count * 16), 256, 0, ctx->stream>>>(
      src, dst, ld_dst, rows, cols);
  HL_LAUNCH_CHECK("rows_f32_to_bf16_kernel");
  count_launch(ctx);
  return HL_OK;
}

int attention_forward_wide(hl_decoder* m, const __nv_bfloat16* qkv, __nv_bfloat16* out) {
  hl_ctx* ctx = m->ctx;
  const hl_decoder_config& c = m->cfg;
  const int N = m->N, d = c.d_model;
  HL_TRY(widen_rows(ctx, qkv, 3 * d, m->fa_q, N, d));
  HL_TRY(widen_rows(ctx, qkv + d, 3 * d, m->fa_k, N, d));
  HL_TRY(widen_rows(ctx, qkv + 2 * d, 3 * d, m->fa_v, N, d));
  HL_TRY(hl_causal_attention_f32_forward(ctx, m->fa_q, m->fa_k, m->fa_v, m->fa_o, m->fa_probs, c.batch, c.context, d, c.n_heads));
  if (out) HL_TRY(narrow_rows(ctx, m->fa_o, out, d, N, d));
  return HL_OK;
}

int attention_backward_wide(hl_decoder* m, const __nv_bfloat16* qkv, const __nv_bfloat16* dout, __nv_bfloat16* dqkv) {
  hl_ctx* ctx = m->ctx;
  const hl_decoder_config& c = m->cfg;
  const int N = m->N, d = c.d_model;
  HL_TRY(attention_forward_wide(m, qkv, nullptr));  // q, k, v and the probabilities again
  HL_TRY(widen_rows(ctx, dout, d, m->fa_do, N, d));
  HL_TRY(hl_causal_attention_f32_backward(ctx, m->fa_q, m->fa_k, m->fa_v, m->fa_probs, m->fa_do, m->fa_dq, m->fa_dk, m->fa_dv,
                                          c.batch, c.context, d, c.n_heads));
  HL_TRY(narrow_rows(ctx, m->fa_dq, dqkv, 3 * d, N, d));
  HL_TRY(narrow_rows(ctx, m->fa_dk, dqkv + d, 3 * d, N, d));
  HL_TRY(narrow_rows(ctx, m->fa_dv, dqkv + 2 * d, 3 * d, N, d));
  return HL_OK;
}

int forward(hl_decoder* m) {
  hl_ctx* ctx = m->ctx;
  const hl_decoder_config& c = m->cfg;
  const int N = m->N, d = c.d_model, F = c.d_ff, V = c.vocab, B = c.batch, T = c.context, H = c.n_heads;
  const Gemm g{m};
  const float* P = m->params;
  const __nv_bfloat16* W = m->shadow;
  if (!m->comm_pending) ctx->reserve_sms = 0;  // nothing of the gradient exchange is in flight during a forward pass
  HL_TRY(hl_embedding_forward(ctx, P + m->off_tok, V, m->tokens, P + m->off_pos, T, m->x[0], HL_BF16, N, d));
  for (int l = 0; l < c.n_layers; ++l) {
    const LayerOffsets& o = m->lo[l];
    LayerActs& a = m->la[l];
    HL_TRY(layer_norm_forward_impl(ctx, m->x[l], HL_BF16, P + o.ln1g, P + o.ln1b, a.a, HL_BF16, a.mean1, a.rstd1, N, d, 1e-5f));
    HL_TRY(g.run(N, 3 * d, d, a.a, d, HL_K_MAJOR, W + o.wqkv, d, HL_K_MAJOR, a.qkv, 3 * d, HL_BF16, HL_EPI_BIAS, P + o.bqkv));
    if (m->flash_ok) HL_TRY(flash_attention_forward_impl(ctx, a.qkv, a.qkv + d, a.qkv + 2 * d, 3 * d, a.o, d, a.lse, B, T, H, d / H));
    else HL_TRY(attention_forward_wide(m, a.qkv, a.o));
    HL_TRY(g.run(N, d, d, a.o, d, HL_K_MAJOR, W + o.wo, d, HL_K_MAJOR, a.r, d, HL_BF16, HL_EPI_BIAS_RESIDUAL, P + o.bo,
                 m->x[l], d));
    HL_TRY(layer_norm_forward_impl(ctx, a.r, HL_BF16, P + o.ln2g, P + o.ln2b, a.c, HL_BF16, a.mean2, a.rstd2, N, d, 1e-5f));
    if (o.is_memory) {
      // The reference keeps the memory feed-forward in f32 under AMP (src/memory_transformer.rs:787-789).  Its three
      // projections still run on the tensor cores here, at f32 accuracy: the block input is bf16-exact, so
      // x*W = x*W_hi + x*W_mid + x*W_lo with exact products and one f32 accumulation (a contraction of 3*d against
      // the weight's three bf16 pieces, the input read three times); out_proj takes the f32 mv as hi + lo pieces and
      // drops only the lo*lo term (2^-16 relative, far below the bf16 rounding of the block output that follows).
      // The query decides the routing, so it has to be this accurate; lookup, scores, softmax, gather and gate are f32.
      MemoryActs& ma = m->ma[l];
      const int kd = m->mem.key_dim, vd = m->mem.value_dim;
      HL_TRY(hl_split_bf16_f32(ctx, P + o.wq_m, ma.wq3, kd, d, HL_SPLIT_HI_MID_LO));
      HL_TRY(hl_split_bf16_f32(ctx, P + o.wg_m, ma.wg3, vd, d, HL_SPLIT_HI_MID_LO));
      HL_TRY(hl_split_bf16_f32(ctx, P + o.wout_m, ma.wout3, d, vd, HL_SPLIT_HI_HI_LO));
      HL_TRY(g.run(N, kd, 3 * d, a.c, d, HL_K_MAJOR, ma.wq3, 3 * d, HL_K_MAJOR, ma.query, kd, HL_F32, HL_EPI_BIAS, P + o.bq_m,
                   nullptr, 0, nullptr, 0, d));
      HL_TRY(memory_core_forward(m, l));
      HL_TRY(g.run(N, vd, 3 * d, a.c, d, HL_K_MAJOR, ma.wg3, 3 * d, HL_K_MAJOR, ma.gpre, vd, HL_F32, HL_EPI_BIAS, P + o.bg_m,
                   nullptr, 0, nullptr, 0, d));
      HL_TRY(hl_gelu(ctx, ma.gpre, ma.gate, HL_F32, (size_t)N * vd));
      HL_TRY(hl_binary_f32(ctx, HL_MUL, ma.weighted, ma.gate, ma.mv, (size_t)N * vd));
      HL_TRY(hl_split_bf16_f32(ctx, ma.mv, ma.mv_b, N, vd, HL_SPLIT_HI_LO));
      HL_TRY(g.run(N, d, 3 * vd, ma.mv_b, 2 * vd, HL_K_MAJOR, ma.wout3, 3 * vd, HL_K_MAJOR, m->x[l + 1], d, HL_BF16,
                   HL_EPI_BIAS_RESIDUAL, P + o.bout_m, a.r, d, nullptr, 0, 2 * vd));
      continue;
    }
    HL_TRY(g.run(N, F, d, a.c, d, HL_K_MAJOR, W + o.w1, d, HL_K_MAJOR, a.h, F, HL_BF16, HL_EPI_BIAS_GELU, P + o.b1, nullptr,
                 0, a.g, F));
    HL_TRY(g.run(N, d, F, a.g, F, HL_K_MAJOR, W + o.w2, F, HL_K_MAJOR, m->x[l + 1], d, HL_BF16, HL_EPI_BIAS_RESIDUAL,
                 P + o.b2, a.r, d));
  }
  HL_TRY(layer_norm_forward_impl(ctx, m->x[c.n_layers], HL_BF16, P + m->off_lnf_g, P + m->off_lnf_b, m->z, HL_BF16, m->meanf,
                                 m->rstdf, N, d, 1e-5f));
  HL_TRY(g.run(N, V, d, m->z, d, HL_K_MAJOR, W + m->off_head_w, d, HL_K_MAJOR, m->logits, V, HL_F32, HL_EPI_BIAS,
               P + m->off_head_b));
  return HL_OK;
}

// Bucket b covers gradient-arena elements [b*bucket, min((b+1)*bucket, arena)); it may be reduced
// once every gradient below its end is final.  Pure host arithmetic, shared with hl_ddp_ready_buckets.
inline void bucket_range(size_t arena, size_t bucket, size_t b, size_t* start, size_t* end) {
  *start = b * bucket;
  *end = std::min(*start + bucket, arena);
}

// Queue the all-reduce of every bucket whose gradients are final.
int flush_buckets(hl_decoder* m, size_t done_elems) {
  if (!nccl_active(m->ctx)) return HL_OK;
  while (m->next_bucket < m->n_buckets) {
    size_t start, end;
    bucket_range(m->arena, m->bucket_elems, m->next_bucket, &start, &end);
    if (end > done_elems) break;
    HL_CUDA(cudaEventRecord(m->bucket_ready[m->next_bucket], m->ctx->stream));
    HL_CUDA(cudaStreamWaitEvent(m->ctx->comm_stream, m->bucket_ready[m->next_bucket], 0));
    // The value table and the token-embedding table travel as the union of the rows that carry a gradient
    // (exchange_rows), not densely: their ranges are cut out of the bucket (value table first, token table last).
    size_t cut_lo[2], cut_hi[2];
    int cuts = 0;
    if (m->has_memory) { cut_lo[cuts] = m->off_val; cut_hi[cuts] = m->off_val + (size_t)m->mem.slots * m->mem.value_dim; ++cuts; }
    if (m->sparse_tok_exchange) { cut_lo[cuts] = m->off_tok; cut_hi[cuts] = m->off_tok + (size_t)m->cfg.vocab * m->cfg.d_model; ++cuts; }
    size_t at = start;
    for (int c = 0; c <= cuts && at < end; ++c) {
      const size_t stop = c < cuts ? std::min(end, std::max(at, cut_lo[c])) : end;
      if (at < stop) HL_TRY(nccl_allreduce_sum_f32(m->ctx, m->grads + at, stop - at, m->ctx->comm_stream));
      at = c < cuts ? std::max(stop, std::min(end, cut_hi[c])) : end;
    }
    HL_CUDA(cudaEventRecord(m->bucket_done[m->next_bucket], m->ctx->comm_stream));
    m->next_bucket += 1;
    m->ctx->reserve_sms = m->ctx->comm_sms;  // collectives are in flight from here to the optimizer's last wait
  }
  return HL_OK;
}

// Data-parallel exchange of a table gradient of which only some rows are non-zero: every rank marks the rows it
// touched, the masks are combined with a byte-wise maximum, the union's gradient rows are packed, summed over the
// ranks and put back (src/bin/heirloom/runtime.rs:4171-4214).  Rows outside the union have zero gradient on every
// rank.  Runs on the collective stream in two halves: the union of the rows when they are known, the exchange of the
// gradient rows after the dense buckets; the host reads the union's size between the two, long after it was written.
struct RowExchange {
  float* grad;            // [rows, dim] in the gradient arena
  int rows, dim;
  unsigned char* flags;   // [rows], zero on entry and on return
  int64_t* union_rows;    // [rows]
  int* count_dev;
  int* count_host;        // pinned
  float** packed;         // own allocation, grown on demand
  size_t* packed_cap;     // rows it holds
  size_t max_events;      // rows all ranks together can touch at most
};

// First half, queued as soon as the touched rows are known: x.flags holds this rank's marks; the union over the ranks, its
// row list and its size (copied to pinned host memory) follow on the collective stream, `ready` after them.
int prepare_rows(hl_decoder* m, const RowExchange& x, cudaEvent_t ready) {
  hl_ctx* ctx = m->ctx;
  cudaStream_t cs = ctx->comm_stream;
  HL_TRY(nccl_allreduce_max_u8(ctx, x.flags, (size_t)x.rows, cs));
  HL_TRY(mask_to_indices_on(ctx, cs, x.flags, x.rows, x.union_rows, x.count_dev));
  HL_CUDA(cudaMemcpyAsync(x.count_host, x.count_dev, sizeof(int), cudaMemcpyDeviceToHost, cs));
  HL_CUDA(cudaMemsetAsync(x.flags, 0, (size_t)x.rows, cs));
  HL_CUDA(cudaEventRecord(ready, cs));
  return HL_OK;
}

// Second half, once the gradient rows are final: pack the union's rows, sum them over the ranks, put them back.  The
// host reads the size here; the device passed `ready` long ago unless the caller queued both halves back to back.
int finish_rows(hl_decoder* m, const RowExchange& x, cudaEvent_t ready, int* union_n) {
  hl_ctx* ctx = m->ctx;
  cudaStream_t cs = ctx->comm_stream;
  HL_CUDA(cudaEventSynchronize(ready));
  const int n = *x.count_host;
  HL_REQUIRE(n >= 0 && n <= x.rows, "hl_decoder: row union out of range");
  *union_n = n;
  if (n > 0) {
    // The packed rows live in a buffer of their own: the context's scratch arena belongs to the compute stream,
    // which keeps running (and may regrow the arena) while this exchange is in flight on the collective stream.
    if ((size_t)n > *x.packed_cap) {
      const size_t cap = std::max((size_t)n, std::min((size_t)x.rows, x.max_events));
      if (*x.packed) {
        HL_CUDA(cudaStreamSynchronize(cs));  // an earlier step's exchange may still be reading the old buffer
        HL_CUDA(cudaFree(*x.packed));
        *x.packed = nullptr;
        *x.packed_cap = 0;
      }
      HL_CUDA(cudaMalloc(reinterpret_cast<void**>(x.packed), sizeof(float) * cap * x.dim));
      *x.packed_cap = cap;
      ctx->counters.allocations += 1;
      ctx->counters.allocated_bytes += sizeof(float) * cap * x.dim;
    }
    HL_TRY(move_rows_on(ctx, cs, x.grad, x.union_rows, nullptr, n, x.dim, *x.packed, false));
    HL_TRY(nccl_allreduce_sum_f32(ctx, *x.packed, (size_t)n * x.dim, cs));
    HL_TRY(move_rows_on(ctx, cs, *x.packed, x.union_rows, nullptr, n, x.dim, x.grad, true));
  }
  return HL_OK;
}

// The value table: rows = the slots the memory blocks selected.
RowExchange value_rows(hl_decoder* m) {
  const size_t per_layer = (size_t)m->N * m->mem.top_k;
  return RowExchange{m->grads + m->off_val, m->mem.slots, m->mem.value_dim, m->m_row_flags, m->m_union_rows, m->m_union_count,
                     m->m_union_count_host, &m->m_packed, &m->packed_rows_cap,
                     (size_t)nccl_world(m->ctx) * per_layer * (size_t)m->mem.n_memory_layers};
}

// Queued after forward: the selections of every memory block are on the device.
int prepare_value_rows(hl_decoder* m) {
  if (!m->has_memory || !nccl_active(m->ctx)) return HL_OK;
  hl_ctx* ctx = m->ctx;
  cudaStream_t cs = ctx->comm_stream;
  const size_t per_layer = (size_t)m->N * m->mem.top_k;
  const int slots = m->mem.slots;
  HL_CUDA(cudaEventRecord(m->rows_known, ctx->stream));
  HL_CUDA(cudaStreamWaitEvent(cs, m->rows_known, 0));
  HL_CUDA(cudaMemsetAsync(m->m_row_flags, 0, (size_t)slots, cs));
  for (int l = 0; l < m->cfg.n_layers; ++l)
    if (m->lo[l].is_memory) HL_TRY(mark_rows_on(ctx, cs, m->ma[l].idx, (long long)per_layer, nullptr, m->m_row_flags, slots));
  HL_TRY(prepare_rows(m, value_rows(m), m->val_count_ready));
  m->val_prepared = true;
  return HL_OK;
}

int exchange_value_rows(hl_decoder* m) {
  if (!m->has_memory || !nccl_active(m->ctx)) return HL_OK;
  if (!m->val_prepared) HL_TRY(prepare_value_rows(m));
  m->val_prepared = false;
  return finish_rows(m, value_rows(m), m->val_count_ready, &m->union_n);
}

// The token-embedding table: rows = the token ids of the batch.  At a Zipf-distributed batch of 16 Ki tokens over a
// vocabulary of 50 Ki this is a small share of the 154 MB table, and it is the gradient that becomes final last in
// backward, i.e. the exchange nothing is left to hide behind.
RowExchange token_rows(hl_decoder* m) {
  return RowExchange{m->grads + m->off_tok, m->cfg.vocab, m->cfg.d_model, m->tok_flags, m->tok_union_rows, m->tok_union_count,
                     m->tok_union_count_host, &m->tok_packed, &m->tok_packed_cap, (size_t)nccl_world(m->ctx) * (size_t)m->N};
}

// Queued as soon as the step's token ids are on the device.
int prepare_token_rows(hl_decoder* m) {
  if (!m->sparse_tok_exchange || !nccl_active(m->ctx)) return HL_OK;
  hl_ctx* ctx = m->ctx;
  cudaStream_t cs = ctx->comm_stream;
  const int V = m->cfg.vocab;
  HL_CUDA(cudaEventRecord(m->rows_known, ctx->stream));
  HL_CUDA(cudaStreamWaitEvent(cs, m->rows_known, 0));
  HL_CUDA(cudaMemsetAsync(m->tok_flags, 0, (size_t)V, cs));
  HL_TRY(mark_rows_on(ctx, cs, m->tokens, (long long)m->N, nullptr, m->tok_flags, V));
  HL_TRY(prepare_rows(m, token_rows(m), m->tok_count_ready));
  m->tok_prepared = true;
  return HL_OK;
}

int exchange_token_rows(hl_decoder* m) {
  if (!m->sparse_tok_exchange || !nccl_active(m->ctx)) return HL_OK;
  if (!m->tok_prepared) HL_TRY(prepare_token_rows(m));
  m->tok_prepared = false;
  int n = 0;
  return finish_rows(m, token_rows(m), m->tok_count_ready, &n);
}

int backward(hl_decoder* m) {
  hl_ctx* ctx = m->ctx;
  const hl_decoder_config& c = m->cfg;
  const int N = m->N, d = c.d_model, F = c.d_ff, V = c.vocab, B = c.batch, T = c.context, H = c.n_heads;
  const Gemm g{m};
  const float* P = m->params;
  const __nv_bfloat16* W = m->shadow;
  float* G = m->grads;
  m->next_bucket = 0;
  if (m->comm_pending) {  // a previous step's collectives were never consumed: finish them before its gradients are overwritten
    HL_CUDA(cudaStreamWaitEvent(m->ctx->stream, m->comm_done, 0));
    m->comm_pending = false;
  }
  HL_TRY(zero_memory_table_grads(m));
  // loss and dlogits = (softmax - onehot)/N in bf16, the operand precision of the next GEMMs
  HL_TRY(cross_entropy_impl(ctx, m->logits, V, m->targets, N, V, 1.0f, m->loss_dev, nullptr, m->dlogits, HL_BF16, V));
  // lm_head
  HL_TRY(g.run(V, d, N, m->dlogits, V, HL_MN_MAJOR, m->z, d, HL_MN_MAJOR, G + m->off_head_w, d, HL_F32));
  FoldBatch* fb = &m->fold;
  fb->n = 0;
  fb->used = 0;
  HL_TRY(bias_grad_impl(ctx, m->dlogits, HL_BF16, G + m->off_head_b, N, V, fb));
  HL_TRY(g.run(N, d, V, m->dlogits, V, HL_K_MAJOR, W + m->off_head_w, d, HL_MN_MAJOR, m->dtmp, d, HL_F32));
  float* dx = m->dx0;
  float* dx_next = m->dx1;
  // every layer-norm backward also returns the column sums of the gradient it writes: the bias
  // gradient of the projection that produced that residual-stream value (fc2 or out_proj)
  HL_TRY(layer_norm_backward_impl(ctx, m->x[c.n_layers], HL_BF16, P + m->off_lnf_g, m->dtmp, m->meanf, m->rstdf, nullptr, dx,
                                  m->dxb, G + m->off_lnf_g, G + m->off_lnf_b, G + m->lo[c.n_layers - 1].out_bias(), N, d, fb));
  HL_TRY(fold_batch_flush(ctx, fb));
  HL_TRY(flush_buckets(m, m->off_lnf_b + d));
  for (int l = c.n_layers - 1; l >= 0; --l) {
    const LayerOffsets& o = m->lo[l];
    LayerActs& a = m->la[l];
    if (o.is_memory) {
      // y = r + out_proj(weighted * gelu(gate_proj(c))), weighted from the lookup on query_proj(c)
      MemoryActs& ma = m->ma[l];
      const int kd = m->mem.key_dim, vd = m->mem.value_dim;
      const size_t nv = (size_t)N * vd;
      // The reference runs these three projections in f32 also backward (src/memory_transformer.rs:787-789).  Here
      // every product stays on the tensor cores with its f32 operands as bf16 pieces: hi*hi + lo*hi + hi*lo in one
      // f32 accumulation (the dropped lo*lo term is 2^-16 relative), or hi + mid + lo (exact) against the block input,
      // which is bf16-exact.  `side`: pieces along the columns, for operands contracted along their rows' direction;
      // `rows`: pieces one below the other, for operands contracted down their rows.
      const int ROWS = HL_SPLIT_STACK_ROWS;
      const float* dy = dx;  // dL/dy of this block, f32
      // out_proj: dW = dy^T mv, dmv = dy W
      HL_TRY(hl_split_bf16_f32(ctx, dy, m->p_dx_rows, N, d, HL_SPLIT_HI_LO | ROWS));
      HL_TRY(hl_split_bf16_f32(ctx, ma.mv, m->p_mv_rows, N, vd, HL_SPLIT_HI_HI_LO | ROWS));
      HL_TRY(g.run(d, vd, 3 * N, m->p_dx_rows, d, HL_MN_MAJOR, m->p_mv_rows, vd, HL_MN_MAJOR, G + o.wout_m, vd, HL_F32,
                   HL_EPI_NONE, nullptr, nullptr, 0, nullptr, 0, 2 * N));
      HL_TRY(hl_split_bf16_f32(ctx, dy, m->p_dx_side, N, d, HL_SPLIT_HI_LO));
      HL_TRY(hl_split_bf16_f32(ctx, P + o.wout_m, m->p_wout_rows, d, vd, HL_SPLIT_HI_HI_LO | ROWS));
      HL_TRY(g.run(N, vd, 3 * d, m->p_dx_side, 2 * d, HL_K_MAJOR, m->p_wout_rows, vd, HL_MN_MAJOR, m->m_dmv, vd, HL_F32,
                   HL_EPI_NONE, nullptr, nullptr, 0, nullptr, 0, 2 * d));
      HL_TRY(hl_binary_f32(ctx, HL_MUL, m->m_dmv, ma.gate, m->m_dweighted, nv));
      HL_TRY(hl_binary_f32(ctx, HL_MUL, m->m_dmv, ma.weighted, m->m_dgate, nv));
      HL_TRY(hl_gelu_backward(ctx, ma.gpre, m->m_dgate, m->m_dgpre, HL_F32, nv));
      // gate_proj: dW = dgpre^T c (c is bf16-exact: three exact pieces of dgpre, c read three times), dc = dgpre W
      HL_TRY(hl_split_bf16_f32(ctx, m->m_dgpre, m->p_dg_rows, N, vd, HL_SPLIT_HI_MID_LO | ROWS));
      HL_TRY(g.run(vd, d, 3 * N, m->p_dg_rows, vd, HL_MN_MAJOR, a.c, d, HL_MN_MAJOR, G + o.wg_m, d, HL_F32, HL_EPI_NONE,
                   nullptr, nullptr, 0, nullptr, 0, 0, N));
      HL_TRY(bias_grad_impl(ctx, m->m_dgpre, HL_F32, G + o.bg_m, N, vd, fb));
      HL_TRY(hl_split_bf16_f32(ctx, m->m_dgpre, m->p_dg_side, N, vd, HL_SPLIT_HI_LO));
      HL_TRY(hl_split_bf16_f32(ctx, P + o.wg_m, m->p_wg_rows, vd, d, HL_SPLIT_HI_HI_LO | ROWS));
      HL_TRY(g.run(N, d, 3 * vd, m->p_dg_side, 2 * vd, HL_K_MAJOR, m->p_wg_rows, d, HL_MN_MAJOR, m->dtmp, d, HL_F32,
                   HL_EPI_NONE, nullptr, nullptr, 0, nullptr, 0, 2 * vd));
      HL_TRY(memory_core_backward(m, l, m->m_dweighted));
      // query_proj: dW = dq^T c, dc += dq W
      HL_TRY(hl_split_bf16_f32(ctx, m->m_dq, m->p_dq_rows, N, kd, HL_SPLIT_HI_MID_LO | ROWS));
      HL_TRY(g.run(kd, d, 3 * N, m->p_dq_rows, kd, HL_MN_MAJOR, a.c, d, HL_MN_MAJOR, G + o.wq_m, d, HL_F32, HL_EPI_NONE,
                   nullptr, nullptr, 0, nullptr, 0, 0, N));
      HL_TRY(bias_grad_impl(ctx, m->m_dq, HL_F32, G + o.bq_m, N, kd, fb));
      HL_TRY(hl_split_bf16_f32(ctx, m->m_dq, m->p_dq_side, N, kd, HL_SPLIT_HI_LO));
      HL_TRY(hl_split_bf16_f32(ctx, P + o.wq_m, m->p_wq_rows, kd, d, HL_SPLIT_HI_HI_LO | ROWS));
      HL_TRY(g.run(N, d, 3 * kd, m->p_dq_side, 2 * kd, HL_K_MAJOR, m->p_wq_rows, d, HL_MN_MAJOR, m->m_dc2, d, HL_F32,
                   HL_EPI_NONE, nullptr, nullptr, 0, nullptr, 0, 2 * kd));
      HL_TRY(hl_binary_f32(ctx, HL_ADD, m->dtmp, m->m_dc2, m->dtmp, (size_t)N * d));
    } else {
    // y = r + fc2(gelu(fc1(c)));   dx is dL/dy (f32), dxb its bf16 operand copy
    HL_TRY(g.run(d, F, N, m->dxb, d, HL_MN_MAJOR, a.g, F, HL_MN_MAJOR, G + o.w2, F, HL_F32));
    HL_TRY(g.run(N, F, d, m->dxb, d, HL_K_MAJOR, W + o.w2, F, HL_MN_MAJOR, m->dh, F, HL_BF16, HL_EPI_DGELU, nullptr, a.h, F));
    HL_TRY(g.run(F, d, N, m->dh, F, HL_MN_MAJOR, a.c, d, HL_MN_MAJOR, G + o.w1, d, HL_F32));
    HL_TRY(bias_grad_impl(ctx, m->dh, HL_BF16, G + o.b1, N, F, fb));
    HL_TRY(g.run(N, d, F, m->dh, F, HL_K_MAJOR, W + o.w1, d, HL_MN_MAJOR, m->dtmp, d, HL_F32));
    }
    // dr = dx + LN2'(dc)
    HL_TRY(layer_norm_backward_impl(ctx, a.r, HL_BF16, P + o.ln2g, m->dtmp, a.mean2, a.rstd2, dx, dx_next, m->dxb,
                                    G + o.ln2g, G + o.ln2b, G + o.bo, N, d, fb));
    std::swap(dx, dx_next);  // dx is now dL/dr
    HL_TRY(g.run(d, d, N, m->dxb, d, HL_MN_MAJOR, a.o, d, HL_MN_MAJOR, G + o.wo, d, HL_F32));
    HL_TRY(g.run(N, d, d, m->dxb, d, HL_K_MAJOR, W + o.wo, d, HL_MN_MAJOR, m->dob, d, HL_BF16));
    if (m->flash_ok) {
      const size_t need = flash_attention_backward_scratch_bytes(B, T, H, d / H);
      if (need > ctx->workspace_bytes) HL_TRY(ensure_workspace(ctx, need));
      HL_TRY(flash_attention_backward_impl(ctx, a.qkv, a.qkv + d, a.qkv + 2 * d, 3 * d, a.o, d, m->dob, d, a.lse, m->dqkv,
                                           m->dqkv + d, m->dqkv + 2 * d, 3 * d, B, T, H, d / H, ctx->workspace,
                                           ctx->workspace_bytes));
    } else {
      HL_TRY(attention_backward_wide(m, a.qkv, m->dob, m->dqkv));
    }
    HL_TRY(g.run(3 * d, d, N, m->dqkv, 3 * d, HL_MN_MAJOR, a.a, d, HL_MN_MAJOR, G + o.wqkv, d, HL_F32));
    HL_TRY(bias_grad_impl(ctx, m->dqkv, HL_BF16, G + o.bqkv, N, 3 * d, fb));
    HL_TRY(g.run(N, d, 3 * d, m->dqkv, 3 * d, HL_K_MAJOR, W + o.wqkv, d, HL_MN_MAJOR, m->dtmp, d, HL_F32));
    // dx_in = dr + LN1'(da)
    HL_TRY(layer_norm_backward_impl(ctx, m->x[l], HL_BF16, P + o.ln1g, m->dtmp, a.mean1, a.rstd1, dx, dx_next, m->dxb,
                                    G + o.ln1g, G + o.ln1b, l > 0 ? G + m->lo[l - 1].out_bias() : nullptr, N, d, fb));
    std::swap(dx, dx_next);
    HL_TRY(fold_batch_flush(ctx, fb));
    HL_TRY(flush_buckets(m, o.ln1b + d));
  }
  // embeddings: scatter-add into zeroed tables
  HL_CUDA(cudaMemsetAsync(G + m->off_pos, 0, sizeof(float) * (m->arena - m->off_pos), ctx->stream));
  HL_TRY(hl_embedding_backward(ctx, dx, m->tokens, G + m->off_tok, V, G + m->off_pos, T, N, d));
  HL_TRY(flush_buckets(m, m->arena));
  if (nccl_active(ctx)) {
    if (m->has_memory || m->sparse_tok_exchange) {
      // the row exchanges read gradients the compute stream is still producing
      HL_CUDA(cudaEventRecord(m->comm_done, ctx->stream));
      HL_CUDA(cudaStreamWaitEvent(ctx->comm_stream, m->comm_done, 0));
      HL_TRY(exchange_token_rows(m));
      HL_TRY(exchange_value_rows(m));
    }
    // The compute stream waits for the collectives only when something reads the averaged gradients:
    // the optimizer takes them bucket group by bucket group, every other reader waits for all of them.
    HL_CUDA(cudaEventRecord(m->comm_done, ctx->comm_stream));
    m->comm_pending = true;
  }
  return HL_OK;
}

// ---- f32 route ---------------------------------------------------------------------------------
// Op by op what the reference's f32 path does (MemoryTransformerLm::forward / loss,
// src/memory_transformer.rs:2069-2081, :1604-1610; Linear = matmul(weight.transpose()) then
// add(bias), src/nn.rs:454-475), every op rounding its f32 result from an f64 accumulation.
hl_matrix_layout dense(long long rows, long long cols) { return hl_matrix_layout{rows, cols, cols, 1, 0}; }
hl_matrix_layout transposed(long long rows, long long cols) { return hl_matrix_layout{cols, rows, 1, cols, 0}; }  // view of [rows, cols] storage

int linear_f32(hl_decoder* m, const float* x, const float* w, const float* b, float* y, int rows, int in, int out) {
  // y = x · Wᵀ (rounded), then + b (rounded)
  const hl_matrix_layout lx = dense(rows, in), lw = transposed(out, in), ly = dense(rows, out);
  HL_TRY(hl_matmul_f32_strided(m->ctx, x, &lx, w, &lw, m->tmp_f, &ly, 0));
  return hl_bias_add_f32(m->ctx, m->tmp_f, b, y, rows, out);
}

int linear_backward_f32(hl_decoder* m, const float* x, const float* w, const float* dy, float* dx, int accumulate_dx,
                        float* dw, float* db, int rows, int in, int out) {
  const hl_matrix_layout ldy = dense(rows, out), lw = dense(out, in), ldx = dense(rows, in);
  if (dx) HL_TRY(hl_matmul_f32_strided(m->ctx, dy, &ldy, w, &lw, dx, &ldx, accumulate_dx));
  const hl_matrix_layout ldyt = transposed(rows, out), lx = dense(rows, in), ldw = dense(out, in);
  HL_TRY(hl_matmul_f32_strided(m->ctx, dy, &ldyt, x, &lx, dw, &ldw, 0));
  return bias_grad_impl(m->ctx, dy, HL_F32, db, rows, out);
}

int forward_f32(hl_decoder* m) {
  hl_ctx* ctx = m->ctx;
  const hl_decoder_config& c = m->cfg;
  const int N = m->N, d = c.d_model, F = c.d_ff, V = c.vocab, B = c.batch, T = c.context, H = c.n_heads;
  const float* P = m->params;
  HL_TRY(hl_embedding_forward(ctx, P + m->off_tok, V, m->tokens, P + m->off_pos, T, m->xf[0], HL_F32, N, d));
  for (int l = 0; l < c.n_layers; ++l) {
    const LayerOffsets& o = m->lo[l];
    hl_decoder::F32Layer& a = m->lf[l];
    HL_TRY(layer_norm_forward_impl(ctx, m->xf[l], HL_F32, P + o.ln1g, P + o.ln1b, a.a, HL_F32, nullptr, nullptr, N, d, 1e-5f));
    HL_TRY(linear_f32(m, a.a, P + o.wqkv, P + o.bqkv, a.q, N, d, d));
    HL_TRY(linear_f32(m, a.a, P + o.wqkv + (size_t)d * d, P + o.bqkv + d, a.k, N, d, d));
    HL_TRY(linear_f32(m, a.a, P + o.wqkv + 2 * (size_t)d * d, P + o.bqkv + 2 * d, a.v, N, d, d));
    HL_TRY(hl_causal_attention_f32_forward(ctx, a.q, a.k, a.v, a.o, a.probs, B, T, d, H));
    HL_TRY(linear_f32(m, a.o, P + o.wo, P + o.bo, a.pr, N, d, d));
    HL_TRY(hl_binary_f32(ctx, HL_ADD, m->xf[l], a.pr, a.r, (size_t)N * d));
    HL_TRY(layer_norm_forward_impl(ctx, a.r, HL_F32, P + o.ln2g, P + o.ln2b, a.c, HL_F32, nullptr, nullptr, N, d, 1e-5f));
    if (o.is_memory) {
      MemoryActs& ma = m->ma[l];
      const int kd = m->mem.key_dim, vd = m->mem.value_dim;
      HL_TRY(linear_f32(m, a.c, P + o.wq_m, P + o.bq_m, ma.query, N, d, kd));
      HL_TRY(memory_core_forward(m, l));
      HL_TRY(linear_f32(m, a.c, P + o.wg_m, P + o.bg_m, ma.gpre, N, d, vd));
      HL_TRY(hl_gelu(ctx, ma.gpre, ma.gate, HL_F32, (size_t)N * vd));
      HL_TRY(hl_binary_f32(ctx, HL_MUL, ma.weighted, ma.gate, ma.mv, (size_t)N * vd));
      HL_TRY(linear_f32(m, ma.mv, P + o.wout_m, P + o.bout_m, a.f, N, vd, d));
    } else {
    HL_TRY(linear_f32(m, a.c, P + o.w1, P + o.b1, a.h, N, d, F));
    HL_TRY(hl_gelu(ctx, a.h, a.g, HL_F32, (size_t)N * F));
    HL_TRY(linear_f32(m, a.g, P + o.w2, P + o.b2, a.f, N, F, d));
    }
    HL_TRY(hl_binary_f32(ctx, HL_ADD, a.r, a.f, m->xf[l + 1], (size_t)N * d));
  }
  HL_TRY(layer_norm_forward_impl(ctx, m->xf[c.n_layers], HL_F32, P + m->off_lnf_g, P + m->off_lnf_b, m->zf, HL_F32, nullptr,
                                 nullptr, N, d, 1e-5f));
  return linear_f32(m, m->zf, P + m->off_head_w, P + m->off_head_b, m->logits, N, d, V);
}

int backward_f32(hl_decoder* m) {
  hl_ctx* ctx = m->ctx;
  const hl_decoder_config& c = m->cfg;
  const int N = m->N, d = c.d_model, F = c.d_ff, V = c.vocab, B = c.batch, T = c.context, H = c.n_heads;
  const float* P = m->params;
  float* G = m->grads;
  m->next_bucket = 0;
  if (m->comm_pending) {  // a previous step's collectives were never consumed: finish them before its gradients are overwritten
    HL_CUDA(cudaStreamWaitEvent(m->ctx->stream, m->comm_done, 0));
    m->comm_pending = false;
  }
  HL_TRY(cross_entropy_impl(ctx, m->logits, V, m->targets, N, V, 1.0f, m->loss_dev, nullptr, m->dlogits_f, HL_F32, V));
  HL_TRY(zero_memory_table_grads(m));
  float* dx = m->d_a;       // gradient of the residual stream
  float* dx_next = m->d_b;
  HL_TRY(linear_backward_f32(m, m->zf, P + m->off_head_w, m->dlogits_f, m->d_c, 0, G + m->off_head_w, G + m->off_head_b, N,
                             d, V));
  HL_TRY(layer_norm_backward_impl(ctx, m->xf[c.n_layers], HL_F32, P + m->off_lnf_g, m->d_c, nullptr, nullptr, nullptr, dx,
                                  nullptr, G + m->off_lnf_g, G + m->off_lnf_b, nullptr, N, d));
  HL_TRY(flush_buckets(m, m->off_lnf_b + d));
  for (int l = c.n_layers - 1; l >= 0; --l) {
    const LayerOffsets& o = m->lo[l];
    hl_decoder::F32Layer& a = m->lf[l];
    if (o.is_memory) {
      MemoryActs& ma = m->ma[l];
      const int kd = m->mem.key_dim, vd = m->mem.value_dim;
      const size_t nv = (size_t)N * vd;
      HL_TRY(linear_backward_f32(m, ma.mv, P + o.wout_m, dx, m->m_dmv, 0, G + o.wout_m, G + o.bout_m, N, vd, d));
      HL_TRY(hl_binary_f32(ctx, HL_MUL, m->m_dmv, ma.gate, m->m_dweighted, nv));
      HL_TRY(hl_binary_f32(ctx, HL_MUL, m->m_dmv, ma.weighted, m->m_dgate, nv));
      HL_TRY(hl_gelu_backward(ctx, ma.gpre, m->m_dgate, m->m_dgpre, HL_F32, nv));
      HL_TRY(linear_backward_f32(m, a.c, P + o.wg_m, m->m_dgpre, m->d_c, 0, G + o.wg_m, G + o.bg_m, N, d, vd));
      HL_TRY(memory_core_backward(m, l, m->m_dweighted));
      // the query path's input gradient is added to the gate path's (rounded sum of two rounded terms)
      HL_TRY(linear_backward_f32(m, a.c, P + o.wq_m, m->m_dq, m->m_dc2, 0, G + o.wq_m, G + o.bq_m, N, d, kd));
      HL_TRY(hl_binary_f32(ctx, HL_ADD, m->d_c, m->m_dc2, m->d_c, (size_t)N * d));
    } else {
    // y = r + fc2(gelu(fc1(ln2 r)))
    HL_TRY(linear_backward_f32(m, a.g, P + o.w2, dx, m->d_wide, 0, G + o.w2, G + o.b2, N, F, d));
    HL_TRY(hl_gelu_backward(ctx, a.h, m->d_wide, m->d_wide2, HL_F32, (size_t)N * F));
    HL_TRY(linear_backward_f32(m, a.c, P + o.w1, m->d_wide2, m->d_c, 0, G + o.w1, G + o.b1, N, d, F));
    }
    HL_TRY(layer_norm_backward_impl(ctx, a.r, HL_F32, P + o.ln2g, m->d_c, nullptr, nullptr, dx, dx_next, nullptr, G + o.ln2g,
                                    G + o.ln2b, nullptr, N, d));
    std::swap(dx, dx_next);  // dL/dr
    // r = x + out_proj(attention(q, k, v))
    HL_TRY(linear_backward_f32(m, a.o, P + o.wo, dx, m->d_c, 0, G + o.wo, G + o.bo, N, d, d));
    HL_TRY(hl_causal_attention_f32_backward(ctx, a.q, a.k, a.v, a.probs, m->d_c, m->d_q, m->d_k, m->d_v, B, T, d, H));
    HL_TRY(linear_backward_f32(m, a.a, P + o.wqkv, m->d_q, m->tmp2_f, 0, G + o.wqkv, G + o.bqkv, N, d, d));
    HL_TRY(linear_backward_f32(m, a.a, P + o.wqkv + (size_t)d * d, m->d_k, m->tmp2_f, 1, G + o.wqkv + (size_t)d * d,
                               G + o.bqkv + d, N, d, d));
    HL_TRY(linear_backward_f32(m, a.a, P + o.wqkv + 2 * (size_t)d * d, m->d_v, m->tmp2_f, 1,
                               G + o.wqkv + 2 * (size_t)d * d, G + o.bqkv + 2 * d, N, d, d));
    HL_TRY(layer_norm_backward_impl(ctx, m->xf[l], HL_F32, P + o.ln1g, m->tmp2_f, nullptr, nullptr, dx, dx_next, nullptr,
                                    G + o.ln1g, G + o.ln1b, nullptr, N, d));
    std::swap(dx, dx_next);
    HL_TRY(flush_buckets(m, o.ln1b + d));
  }
  HL_CUDA(cudaMemsetAsync(G + m->off_pos, 0, sizeof(float) * (m->arena - m->off_pos), ctx->stream));
  HL_TRY(hl_embedding_backward(ctx, dx, m->tokens, G + m->off_tok, V, G + m->off_pos, T, N, d));
  HL_TRY(flush_buckets(m, m->arena));
  if (nccl_active(ctx)) {
    if (m->has_memory || m->sparse_tok_exchange) {
      // the row exchanges read gradients the compute stream is still producing
      HL_CUDA(cudaEventRecord(m->comm_done, ctx->stream));
      HL_CUDA(cudaStreamWaitEvent(ctx->comm_stream, m->comm_done, 0));
      HL_TRY(exchange_token_rows(m));
      HL_TRY(exchange_value_rows(m));
    }
    // The compute stream waits for the collectives only when something reads the averaged gradients:
    // the optimizer takes them bucket group by bucket group, every other reader waits for all of them.
    HL_CUDA(cudaEventRecord(m->comm_done, ctx->comm_stream));
    m->comm_pending = true;
  }
  return HL_OK;
}

// The compute stream waits for `ev` of the collective stream.  With per-kernel timing on, the wait is bracketed by two
// timing events: the first completes when the compute stream has run dry, the second when the collective has arrived,
// so their distance is the time this wait left the GPU's compute stream idle.
int wait_on_collective(hl_decoder* m, cudaEvent_t ev) {
  cudaStream_t s = m->ctx->stream;
  const bool timed = m->ctx->profiler != nullptr;
  if (timed) {
    if (m->waits_recorded == m->wait_begin.size()) {
      cudaEvent_t a = nullptr, b = nullptr;
      HL_CUDA(cudaEventCreate(&a));
      HL_CUDA(cudaEventCreate(&b));
      m->wait_begin.push_back(a);
      m->wait_end.push_back(b);
    }
    HL_CUDA(cudaEventRecord(m->wait_begin[m->waits_recorded], s));
  }
  HL_CUDA(cudaStreamWaitEvent(s, ev, 0));
  if (timed) {
    HL_CUDA(cudaEventRecord(m->wait_end[m->waits_recorded], s));
    m->waits_recorded += 1;
  }
  return HL_OK;
}

// Make the compute stream wait for every gradient collective of the step.
int wait_for_collectives(hl_decoder* m) {
  if (m->comm_pending) {
    HL_TRY(wait_on_collective(m, m->comm_done));
    m->comm_pending = false;
  }
  m->ctx->reserve_sms = 0;
  return HL_OK;
}

int optimizer_step(hl_decoder* m) {
  HL_REQUIRE(m->has_opt, "hl_decoder: no optimizer configured (call hl_decoder_set_optimizer)");
  hl_ctx* ctx = m->ctx;
  if (m->opt.clip_norm > 0.f) HL_TRY(wait_for_collectives(m));  // the global norm needs every averaged gradient
  const int world = nccl_world(ctx);
  const float inv_world = 1.0f / (float)world;  // sum then scale by 1/world (src/nn.rs:2100-2117)
  double clip = 1.0;
  if (m->opt.clip_norm > 0.f) {
    // global gradient norm after averaging; forces one device-to-host read like the reference
    HL_TRY(hl_sum_squares_f32(ctx, m->grads, m->arena, m->norm_dev));
    HL_CUDA(cudaMemcpyAsync(m->norm_host, m->norm_dev, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    HL_CUDA(cudaStreamSynchronize(ctx->stream));
    const double sum_sq = (double)m->norm_host[0] * (double)inv_world * (double)inv_world;
    if (!(sum_sq >= 0.0) || sum_sq > 1e300) return fail("non-finite or negative global gradient sum-of-squares");
    const double norm = sqrt(sum_sq);
    if (norm > (double)m->opt.clip_norm) clip = (double)m->opt.clip_norm / (norm + 1e-12);
  }
  m->step += 1;
  hl_adamw_params hp{};
  hp.lr = m->opt.lr; hp.beta1 = m->opt.beta1; hp.beta2 = m->opt.beta2; hp.eps = m->opt.eps;
  hp.weight_decay = m->opt.weight_decay;
  hp.clip_scale = (float)clip * inv_world;
  hp.bias_correction1 = (float)(1.0 - pow((double)m->opt.beta1, (double)m->step));
  hp.bias_correction2 = (float)(1.0 - pow((double)m->opt.beta2, (double)m->step));
  if (!m->comm_pending) return adam_plan_step(ctx, m->plan, &hp);
  // Collectives still in flight: update the arena in groups of buckets, each group as soon as its last
  // all-reduce has finished, so the update of the early buckets overlaps the reduction of the late ones.
  const size_t chunk = (size_t)adam_plan_chunk_elements();
  const int chunks_total = adam_plan_chunk_count(m->plan);
  constexpr size_t kGroup = 5;  // buckets per launch
  int first = 0;
  for (size_t b0 = 0; b0 < m->n_buckets; b0 += kGroup) {
    const size_t b1 = std::min(b0 + kGroup, m->n_buckets);
    size_t start, end;
    bucket_range(m->arena, m->bucket_elems, b1 - 1, &start, &end);
    // chunks that lie completely inside the buckets reduced so far (a chunk that straddles the boundary waits
    // for the next group; the last group takes everything that is left)
    const int upto = b1 == m->n_buckets ? chunks_total : (int)(end / chunk);
    // The gradients of the value table and of the token-embedding table are not final when their buckets are: their
    // rows are summed over the ranks by the row exchanges that follow the last bucket on the collective stream.  A
    // group that reaches into such a table waits for the end of that stream's work (which covers every bucket too).
    const size_t range_end = b1 == m->n_buckets ? m->arena : (size_t)upto * chunk;
    const bool reaches_values = (m->has_memory && range_end > m->off_val) || (m->sparse_tok_exchange && range_end > m->off_tok);
    HL_TRY(wait_on_collective(m, reaches_values ? m->comm_done : m->bucket_done[b1 - 1]));
    HL_TRY(adam_plan_step_range(ctx, m->plan, &hp, first, upto - first));
    first = upto;
  }
  m->comm_pending = false;
  ctx->reserve_sms = 0;
  return HL_OK;
}

int refresh_shadow(hl_decoder* m, size_t offset, size_t numel) {
  return hl_cast(m->ctx, m->params + offset, HL_F32, m->shadow + offset, HL_BF16, numel);
}

}  // namespace
}  // namespace hl

extern "C" {

static int decoder_create_impl(hl_ctx* ctx, const hl_decoder_config* cfg, const hl_memory_config* mem, hl_decoder** out);

int hl_decoder_create(hl_ctx* ctx, const hl_decoder_config* cfg, hl_decoder** out) {
  return decoder_create_impl(ctx, cfg, nullptr, out);
}

int hl_memory_decoder_create(hl_ctx* ctx, const hl_decoder_config* cfg, const hl_memory_config* mem, hl_decoder** out) {
  HL_REQUIRE(mem, "hl_memory_decoder_create: null memory configuration");
  return decoder_create_impl(ctx, cfg, mem, out);
}

int hl_decoder_selected_indices(hl_decoder* m, int layer, int64_t* host, long long count) {
  HL_REQUIRE(m && host, "hl_decoder_selected_indices: null argument");
  HL_REQUIRE(m->has_memory && layer >= 0 && layer < m->cfg.n_layers && m->lo[layer].is_memory,
             "hl_decoder_selected_indices: block " + std::to_string(layer) + " has no memory feed-forward");
  HL_REQUIRE(count == (long long)m->N * m->mem.top_k, "hl_decoder_selected_indices: expected tokens * top_k entries");
  return hl_memory_copy_indices(m->ctx, host, m->ma[layer].idx, count);
}

static int decoder_create_impl(hl_ctx* ctx, const hl_decoder_config* cfg, const hl_memory_config* mem, hl_decoder** out) {
  HL_REQUIRE(ctx && cfg && out, "hl_decoder_create: null argument");
  *out = nullptr;
  int side = 0;
  if (mem && mem->n_memory_layers > 0) {
    HL_REQUIRE(mem->n_memory_layers <= 16, "hl_memory_decoder_create: at most 16 memory layers");
    for (int i = 0; i < mem->n_memory_layers; ++i)
      HL_REQUIRE(mem->memory_layers[i] >= 0 && mem->memory_layers[i] < cfg->n_layers,
                 "hl_memory_decoder_create: memory layer index out of range");
    HL_REQUIRE(mem->slots > 0 && mem->key_dim > 0 && mem->value_dim > 0 && mem->top_k > 0,
               "hl_memory_decoder_create: memory sizes must be positive");
    side = (int)sqrt((double)mem->slots);
    HL_REQUIRE((long long)side * side == mem->slots,
               "product-key memory lookup requires square memory_slots, got " + std::to_string(mem->slots));
    HL_REQUIRE(mem->key_dim % 2 == 0, "product-key memory lookup requires even memory_key_dim, got " + std::to_string(mem->key_dim));
    HL_REQUIRE(mem->memory_heads == 1, "memory_heads=" + std::to_string(mem->memory_heads) +
                                           " requested, but the memory feed-forward supports one memory head");
    HL_REQUIRE(mem->value_dim % 8 == 0 && mem->key_dim % 8 == 0, "hl_memory_decoder_create: key_dim and value_dim must be multiples of 8");
    HL_REQUIRE(side <= 2048 && mem->top_k <= 1024, "hl_memory_decoder_create: side <= 2048 and top_k <= 1024");
  }
  HL_REQUIRE(cfg->vocab > 0 && cfg->d_model > 0 && cfg->n_layers > 0 && cfg->n_heads > 0 && cfg->d_ff > 0 &&
                 cfg->context > 0 && cfg->batch > 0,
             "hl_decoder_create: every size must be positive");
  HL_REQUIRE(cfg->d_model % cfg->n_heads == 0, "hl_decoder_create: d_model must be divisible by n_heads");
  HL_REQUIRE(cfg->precision == HL_PRECISION_AMP_BF16 || cfg->precision == HL_PRECISION_F32,
             "hl_decoder_create: precision must be HL_PRECISION_F32 or HL_PRECISION_AMP_BF16");
  const bool amp = cfg->precision == HL_PRECISION_AMP_BF16;
  if (amp) {
    HL_REQUIRE(cfg->d_model % 8 == 0 && cfg->d_ff % 8 == 0 && cfg->vocab % 8 == 0 && cfg->d_model <= 1024,
               "hl_decoder_create: d_model (<= 1024), d_ff and vocab must be multiples of 8");
    if (mem && mem->n_memory_layers > 0)  // the projections' contraction is read piecewise in whole 64-element blocks
      HL_REQUIRE(cfg->d_model % 64 == 0 && mem->value_dim % 32 == 0 && mem->key_dim % 32 == 0 &&
                     (cfg->batch * cfg->context) % 64 == 0,
                 "hl_memory_decoder_create: the bf16 route needs d_model and batch*context to be multiples of 64, "
                 "key_dim and value_dim of 32");
  } else {
    HL_REQUIRE(cfg->d_model % 4 == 0 && cfg->d_model <= 1024,
               "hl_decoder_create: the f32 route needs d_model to be a multiple of 4 and at most 1024");
  }
  hl_decoder* m = new hl_decoder();
  m->ctx = ctx;
  m->cfg = *cfg;
  m->N = cfg->batch * cfg->context;
  m->flash_ok = cfg->d_model / cfg->n_heads == 64 || cfg->d_model / cfg->n_heads == 128;
  if (mem && mem->n_memory_layers > 0) {
    m->has_memory = true;
    m->mem = *mem;
    m->side = side;
  }
  plan_parameters(m);
  auto cleanup = [&](int rc) { hl_decoder_destroy(m); return rc; };
  cudaError_t e;
  const size_t fb = sizeof(float) * m->arena;
#define HL_ALLOC(ptr, bytes)                                              \
  e = cudaMalloc(reinterpret_cast<void**>(&(ptr)), (bytes));               \
  if (e != cudaSuccess) return cleanup(fail_cuda(e, "cudaMalloc(" #ptr ")"));
  HL_ALLOC(m->params, fb)
  HL_ALLOC(m->grads, fb)
  HL_ALLOC(m->m, fb)
  HL_ALLOC(m->v, fb)
  HL_ALLOC(m->shadow, sizeof(__nv_bfloat16) * m->arena)
  size_t act = 0;
  if (amp) plan_activations(m, true, &act); else plan_activations_f32(m, true, &act);
  m->act_bytes = act;
  HL_ALLOC(m->act_arena, act)
#undef HL_ALLOC
  if (amp) plan_activations(m, false, &act); else plan_activations_f32(m, false, &act);
  cudaMemsetAsync(m->params, 0, fb, ctx->stream);
  cudaMemsetAsync(m->grads, 0, fb, ctx->stream);
  cudaMemsetAsync(m->m, 0, fb, ctx->stream);
  cudaMemsetAsync(m->v, 0, fb, ctx->stream);
  cudaMemsetAsync(m->shadow, 0, sizeof(__nv_bfloat16) * m->arena, ctx->stream);
  e = cudaMallocHost(reinterpret_cast<void**>(&m->loss_host), 64);
  if (e != cudaSuccess) return cleanup(fail_cuda(e, "cudaMallocHost"));
  m->norm_host = m->loss_host + 8;
  m->m_union_count_host = reinterpret_cast<int*>(m->loss_host + 12);
  m->tok_union_count_host = reinterpret_cast<int*>(m->loss_host + 13);
  if (const char* e = getenv("HEIRLOOM_SPARSE_EMBEDDING_EXCHANGE")) m->sparse_tok_exchange = atoi(e) != 0;
  hl_adamw_tensor whole{m->params, m->grads, m->m, m->v, m->shadow, (uint64_t)m->arena};
  int rc = adam_plan_create(ctx, &whole, 1, &m->plan);
  if (rc != HL_OK) return cleanup(rc);
  if (m->has_memory) {
    auto span = [&](size_t begin, size_t end) {
      return hl_adamw_tensor{m->params + begin, m->grads + begin, m->m + begin, m->v + begin, m->shadow + begin,
                             (uint64_t)(end - begin)};
    };
    hl_adamw_tensor tables = span(m->off_kl, m->tables_end);
    rc = adam_plan_create(ctx, &tables, 1, &m->plan_tables);
    if (rc != HL_OK) return cleanup(rc);
    hl_adamw_tensor rest[2] = {span(0, m->off_val), span(m->tables_end, m->arena)};
    rc = adam_plan_create(ctx, rest, 2, &m->plan_no_values);
    if (rc != HL_OK) return cleanup(rc);
  }
  m->n_buckets = (m->arena + m->bucket_elems - 1) / m->bucket_elems;
  m->bucket_ready.resize(m->n_buckets);
  m->bucket_done.resize(m->n_buckets);
  for (auto& ev : m->bucket_done) {
    cudaError_t ee = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (ee != cudaSuccess) { ev = nullptr; return fail_cuda(ee, "cudaEventCreate(bucket_done)"); }
  }
  for (auto& ev : m->bucket_ready) {
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return cleanup(fail_cuda(e, "cudaEventCreate"));
  }
  for (cudaEvent_t* ev : {&m->rows_known, &m->tok_count_ready, &m->val_count_ready}) {
    e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
    if (e != cudaSuccess) { *ev = nullptr; return fail_cuda(e, "cudaEventCreate(row exchange)"); }
  }
  e = cudaEventCreateWithFlags(&m->comm_done, cudaEventDisableTiming);
  if (e != cudaSuccess) return cleanup(fail_cuda(e, "cudaEventCreate"));
  e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) return cleanup(fail_cuda(e, "cudaStreamSynchronize"));
  ctx->counters.allocations += 6;
  ctx->counters.allocated_bytes += 4 * fb + sizeof(__nv_bfloat16) * m->arena + act;
  *out = m;
  return HL_OK;
}

void hl_decoder_destroy(hl_decoder* m) {
  if (!m) return;
  if (m->ctx) {
    cudaStreamSynchronize(m->ctx->stream);
    cudaStreamSynchronize(m->ctx->comm_stream);
  }
  for (auto ev : m->bucket_ready) if (ev) cudaEventDestroy(ev);
  for (auto ev : m->bucket_done) if (ev) cudaEventDestroy(ev);
  if (m->comm_done) cudaEventDestroy(m->comm_done);
  for (cudaEvent_t ev : {m->rows_known, m->tok_count_ready, m->val_count_ready}) if (ev) cudaEventDestroy(ev);
  for (auto ev : m->wait_begin) cudaEventDestroy(ev);
  for (auto ev : m->wait_end) cudaEventDestroy(ev);
  adam_plan_destroy(m->plan);
  adam_plan_destroy(m->plan_tables);
  adam_plan_destroy(m->plan_no_values);
  if (m->m_packed) cudaFree(m->m_packed);
  if (m->tok_packed) cudaFree(m->tok_packed);
  cudaFree(m->params); cudaFree(m->grads); cudaFree(m->m); cudaFree(m->v); cudaFree(m->shadow); cudaFree(m->act_arena);
  if (m->loss_host) cudaFreeHost(m->loss_host);
  delete m;
}

int hl_decoder_param_count(hl_decoder* m) { return m ? (int)m->slots.size() : 0; }

int hl_decoder_param_info(hl_decoder* m, int index, char* name_out, size_t name_cap, long long* numel, int* rank,
                          long long shape_out[2]) {
  HL_REQUIRE(m, "hl_decoder_param_info: null model");
  HL_REQUIRE(index >= 0 && index < (int)m->slots.size(), "hl_decoder_param_info: parameter index out of range");
  const Slot& s = m->slots[index];
  if (name_out && name_cap > 0) {
    strncpy(name_out, s.name.c_str(), name_cap - 1);
    name_out[name_cap - 1] = 0;
  }
  if (numel) *numel = (long long)s.numel;
  if (rank) *rank = s.rank;
  if (shape_out) { shape_out[0] = s.shape[0]; shape_out[1] = s.shape[1]; }
  return HL_OK;
}

static int slot_io(hl_decoder* m, int index, long long numel, const Slot** out, const char* who) {
  HL_REQUIRE(m, std::string(who) + ": null model");
  HL_REQUIRE(index >= 0 && index < (int)m->slots.size(), std::string(who) + ": parameter index out of range");
  const Slot& s = m->slots[index];
  HL_REQUIRE(numel == (long long)s.numel, std::string(who) + ": parameter " + s.name + " has " + std::to_string(s.numel) +
                                              " elements, got " + std::to_string(numel));
  *out = &s;
  return HL_OK;
}

int hl_decoder_set_param(hl_decoder* m, int index, const float* host, long long numel) {
  const Slot* s;
  HL_TRY(slot_io(m, index, numel, &s, "hl_decoder_set_param"));
  HL_TRY(hl_memcpy_h2d(m->ctx, m->params + s->offset, host, sizeof(float) * s->numel));
  return refresh_shadow(m, s->offset, s->numel);
}

int hl_decoder_get_param(hl_decoder* m, int index, float* host, long long numel) {
  const Slot* s;
  HL_TRY(slot_io(m, index, numel, &s, "hl_decoder_get_param"));
  return hl_memcpy_d2h(m->ctx, host, m->params + s->offset, sizeof(float) * s->numel);
}

int hl_decoder_get_grad(hl_decoder* m, int index, float* host, long long numel) {
  const Slot* s;
  HL_TRY(slot_io(m, index, numel, &s, "hl_decoder_get_grad"));
  HL_TRY(hl::wait_for_collectives(m));
  return hl_memcpy_d2h(m->ctx, host, m->grads + s->offset, sizeof(float) * s->numel);
}

int hl_decoder_get_moments(hl_decoder* m, int index, float* m_host, float* v_host, long long numel) {
  const Slot* s;
  HL_TRY(slot_io(m, index, numel, &s, "hl_decoder_get_moments"));
  HL_TRY(hl_memcpy_d2h(m->ctx, m_host, m->m + s->offset, sizeof(float) * s->numel));
  return hl_memcpy_d2h(m->ctx, v_host, m->v + s->offset, sizeof(float) * s->numel);
}

int hl_decoder_set_optimizer(hl_decoder* m, const hl_adamw_config* opt) {
  HL_REQUIRE(m && opt, "hl_decoder_set_optimizer: null argument");
  HL_REQUIRE(opt->lr >= 0.f && opt->beta1 >= 0.f && opt->beta1 < 1.f && opt->beta2 >= 0.f && opt->beta2 < 1.f &&
                 opt->eps > 0.f && opt->weight_decay >= 0.f,
             "hl_decoder_set_optimizer: invalid AdamW hyper-parameters");
  m->opt = *opt;
  m->has_opt = true;
  m->step = 0;
  HL_CUDA(cudaMemsetAsync(m->m, 0, sizeof(float) * m->arena, m->ctx->stream));
  HL_CUDA(cudaMemsetAsync(m->v, 0, sizeof(float) * m->arena, m->ctx->stream));
  return HL_OK;
}

long long hl_decoder_optimizer_steps(hl_decoder* m) { return m ? m->step : 0; }

int hl_decoder_set_moments(hl_decoder* m, int index, const float* m_host, const float* v_host, long long numel) {
  const Slot* s;
  HL_TRY(slot_io(m, index, numel, &s, "hl_decoder_set_moments"));
  HL_REQUIRE(m_host && v_host, "hl_decoder_set_moments: null argument");
  HL_REQUIRE(m->has_opt, "hl_decoder_set_moments: no optimizer configured (call hl_decoder_set_optimizer)");
  HL_TRY(hl_memcpy_h2d(m->ctx, m->m + s->offset, m_host, sizeof(float) * s->numel));
  return hl_memcpy_h2d(m->ctx, m->v + s->offset, v_host, sizeof(float) * s->numel);
}

int hl_decoder_set_optimizer_steps(hl_decoder* m, long long steps) {
  HL_REQUIRE(m, "hl_decoder_set_optimizer_steps: null model");
  HL_REQUIRE(m->has_opt, "hl_decoder_set_optimizer_steps: no optimizer configured (call hl_decoder_set_optimizer)");
  HL_REQUIRE(steps >= 0, "hl_decoder_set_optimizer_steps: the step counter cannot be negative");
  m->step = steps;
  return HL_OK;
}

int hl_decoder_forward_backward(hl_decoder* m, const int64_t* tokens_dev, const int64_t* targets_dev) {
  HL_REQUIRE(m && tokens_dev && targets_dev, "hl_decoder_forward_backward: null argument");
  const unsigned long long before = m->ctx->counters.launches;
  if (tokens_dev != m->tokens)
    HL_CUDA(cudaMemcpyAsync(m->tokens, tokens_dev, sizeof(int64_t) * m->N, cudaMemcpyDeviceToDevice, m->ctx->stream));
  if (targets_dev != m->targets)
    HL_CUDA(cudaMemcpyAsync(m->targets, targets_dev, sizeof(int64_t) * m->N, cudaMemcpyDeviceToDevice, m->ctx->stream));
  HL_TRY(prepare_token_rows(m));  // data parallel: the union of the ranks' token rows forms while forward runs
  if (m->cfg.precision == HL_PRECISION_AMP_BF16) {
    HL_TRY(forward(m));
    HL_TRY(prepare_value_rows(m));
    HL_TRY(backward(m));
  } else {
    HL_TRY(forward_f32(m));
    HL_TRY(prepare_value_rows(m));
    HL_TRY(backward_f32(m));
  }
  m->launches_last_step = m->ctx->counters.launches - before;
  return HL_OK;
}

int hl_decoder_optimizer_step(hl_decoder* m) {
  HL_REQUIRE(m, "hl_decoder_optimizer_step: null model");
  const unsigned long long before = m->ctx->counters.launches;
  HL_TRY(optimizer_step(m));
  m->launches_last_step += m->ctx->counters.launches - before;
  return HL_OK;
}

namespace hl {
namespace {

constexpr int kTableLeft = 1, kTableRight = 2, kTableValue = 4, kTablesAll = 7;

// The rows the sparse policies work on, as one list for all memory blocks (a row chosen by several blocks or tokens
// is updated once; memory_sparse_adamw_updates, src/memory_transformer.rs:1293-1424), split into the half-key rows.
// Under data parallelism the list is the union over the ranks, formed by the exchange at the end of backward:
// every rank updates the rows any rank selected, with the averaged gradient (src/bin/heirloom/runtime.rs:4171-4214).
int gather_selection(hl_decoder* m, size_t* total_out) {
  hl_ctx* ctx = m->ctx;
  const size_t per_layer = (size_t)m->N * m->mem.top_k;
  size_t total = 0;
  if (nccl_active(ctx)) {
    HL_REQUIRE(m->union_n >= 0, "hl_decoder: sparse-row update requested, but no backward pass has run yet");
    HL_TRY(wait_for_collectives(m));
    total = (size_t)m->union_n;
    HL_CUDA(cudaMemcpyAsync(m->m_sel_all, m->m_union_rows, sizeof(int64_t) * total, cudaMemcpyDeviceToDevice, ctx->stream));
  } else {
    for (int l = 0; l < m->cfg.n_layers; ++l) {
      if (!m->lo[l].is_memory) continue;
      HL_CUDA(cudaMemcpyAsync(m->m_sel_all + total, m->ma[l].idx, sizeof(int64_t) * per_layer, cudaMemcpyDeviceToDevice,
                              ctx->stream));
      total += per_layer;
    }
  }
  if (total > 0) HL_TRY(hl_product_key_split_rows(ctx, m->m_sel_all, m->m_sel_left, m->m_sel_right, (long long)total, m->side));
  *total_out = total;
  return HL_OK;
}

struct SparseTable {
  size_t offset;
  const int64_t* rows;
  const unsigned char* mask;
  int n_rows, row_dim;
};

// SMFT: a table row is updated only where its mask allows (memory_sparse_adamw_updates_with_mask,
// src/memory_transformer.rs:1426-1468)
void sparse_tables(hl_decoder* m, int which, SparseTable out[3], int* count) {
  const int half = m->mem.key_dim / 2;
  int n = 0;
  if (which & kTableLeft) out[n++] = {m->off_kl, m->m_sel_left, m->smft_on ? m->smft_left_mask : nullptr, m->side, half};
  if (which & kTableRight) out[n++] = {m->off_kr, m->m_sel_right, m->smft_on ? m->smft_right_mask : nullptr, m->side, half};
  if (which & kTableValue)
    out[n++] = {m->off_val, m->m_sel_all, m->smft_on ? m->smft_value_mask : nullptr, m->mem.slots, m->mem.value_dim};
  *count = n;
}

// adds the sum of squares of the active rows of the chosen tables to *sum_dev (f64, on the device)
int sparse_sum_squares(hl_decoder* m, size_t total, int which, double* sum_dev) {
  SparseTable t[3];
  int n = 0;
  sparse_tables(m, which, t, &n);
  for (int i = 0; i < n; ++i)
    HL_TRY(hl_sparse_rows_sum_squares_f32(m->ctx, m->grads + t[i].offset, t[i].rows, (long long)total, t[i].mask,
                                          m->m_row_flags, t[i].n_rows, t[i].row_dim, sum_dev));
  return HL_OK;
}

int sparse_adamw(hl_decoder* m, size_t total, int which, const hl_adamw_params& hp) {
  SparseTable t[3];
  int n = 0;
  sparse_tables(m, which, t, &n);
  for (int i = 0; i < n; ++i)
    HL_TRY(hl_sparse_adamw_rows_f32(m->ctx, m->params + t[i].offset, m->grads + t[i].offset, m->m + t[i].offset,
                                    m->v + t[i].offset, t[i].rows, (long long)total, t[i].mask, m->m_row_flags, t[i].n_rows,
                                    t[i].row_dim, &hp, 0));
  return HL_OK;
}

hl_adamw_params step_params(hl_decoder* m, double clip) {
  hl_adamw_params hp{};
  hp.lr = m->opt.lr; hp.beta1 = m->opt.beta1; hp.beta2 = m->opt.beta2; hp.eps = m->opt.eps;
  hp.weight_decay = m->opt.weight_decay;
  hp.clip_scale = (float)clip * (1.0f / (float)nccl_world(m->ctx));  // summed gradients are averaged (src/nn.rs:2100-2117)
  hp.bias_correction1 = (float)(1.0 - pow((double)m->opt.beta1, (double)m->step));
  hp.bias_correction2 = (float)(1.0 - pow((double)m->opt.beta2, (double)m->step));
  return hp;
}

// clip factor from a sum of squares of summed (not yet averaged) gradients
int clip_from_sum(hl_decoder* m, double sum_sq, const char* what, double* clip) {
  *clip = 1.0;
  if (!(sum_sq >= 0.0) || sum_sq > 1e300) return fail(std::string("non-finite or negative ") + what + " sum-of-squares");
  const double norm = sqrt(sum_sq) / (double)nccl_world(m->ctx);  // norm of the averaged gradient
  if (norm > (double)m->opt.clip_norm) *clip = (double)m->opt.clip_norm / (norm + 1e-12);
  return HL_OK;
}

int step_sparse_rows(hl_decoder* m) {
  hl_ctx* ctx = m->ctx;
  size_t total = 0;
  HL_TRY(gather_selection(m, &total));
  if (total == 0) { m->step += 1; return HL_OK; }
  m->step += 1;  // every sparse call advances the step counter (src/nn.rs:2262)
  HL_CUDA(cudaMemsetAsync(m->m_row_flags, 0, (size_t)m->mem.slots, ctx->stream));
  double clip = 1.0;
  if (m->opt.clip_norm > 0.f) {
    // norm over the active rows of the three tables only (clip_scale_for_sparse_row_updates, src/nn.rs:2667-2774)
    HL_CUDA(cudaMemsetAsync(m->norm_dev64, 0, sizeof(double), ctx->stream));
    HL_TRY(sparse_sum_squares(m, total, kTablesAll, m->norm_dev64));
    double sum_sq = 0.0;
    HL_TRY(hl_memcpy_d2h(ctx, &sum_sq, m->norm_dev64, sizeof(double)));
    HL_TRY(clip_from_sum(m, sum_sq, "sparse selected gradient", &clip));
  }
  return sparse_adamw(m, total, kTablesAll, step_params(m, clip));
}

// `MemoryOnly` (src/bin/heirloom/runtime.rs:2440-2450; AdamW::step_parameter_indices_mut, src/nn.rs:2222-2254):
// dense AdamW on the memory tables alone, clip norm over those tables.
int step_memory_only(hl_decoder* m) {
  hl_ctx* ctx = m->ctx;
  HL_TRY(wait_for_collectives(m));
  const size_t begin = m->off_kl, n = m->tables_end - m->off_kl;
  double clip = 1.0;
  if (m->opt.clip_norm > 0.f) {
    HL_TRY(hl_sum_squares_f32(ctx, m->grads + begin, n, m->norm_dev));
    float sum = 0.f;
    HL_TRY(hl_memcpy_d2h(ctx, &sum, m->norm_dev, sizeof(float)));
    HL_TRY(clip_from_sum(m, (double)sum, "memory table gradient", &clip));
  }
  m->step += 1;
  const hl_adamw_params hp = step_params(m, clip);
  return adam_plan_step(ctx, m->plan_tables, &hp);
}

// Dense AdamW everywhere except the value table, row-set AdamW on the value rows the step selected: one step count,
// one clip factor from the dense gradients plus the active value rows.  The value table (slots x value_dim) is by
// far the largest parameter and only tokens*top_k of its rows carry a gradient, so this skips both the dense pass
// over it and the decay of rows nobody read.
int step_dense_plus_sparse_values(hl_decoder* m) {
  hl_ctx* ctx = m->ctx;
  size_t total = 0;
  HL_TRY(gather_selection(m, &total));  // waits for the collectives under data parallelism
  HL_CUDA(cudaMemsetAsync(m->m_row_flags, 0, (size_t)m->mem.slots, ctx->stream));
  double clip = 1.0;
  if (m->opt.clip_norm > 0.f) {
    const size_t tail = m->tables_end, tail_n = m->arena - m->tables_end;
    HL_TRY(hl_sum_squares_f32(ctx, m->grads, m->off_val, m->norm_dev));
    HL_TRY(hl_sum_squares_f32(ctx, m->grads + tail, tail_n, m->norm_dev + 1));
    HL_CUDA(cudaMemsetAsync(m->norm_dev64, 0, sizeof(double), ctx->stream));
    if (total > 0) HL_TRY(sparse_sum_squares(m, total, kTableValue, m->norm_dev64));
    float dense[2] = {0.f, 0.f};
    double rows = 0.0;
    HL_TRY(hl_memcpy_d2h(ctx, dense, m->norm_dev, sizeof(dense)));
    HL_TRY(hl_memcpy_d2h(ctx, &rows, m->norm_dev64, sizeof(double)));
    HL_TRY(clip_from_sum(m, (double)dense[0] + (double)dense[1] + rows, "gradient", &clip));
  }
  m->step += 1;
  const hl_adamw_params hp = step_params(m, clip);
  HL_TRY(adam_plan_step(ctx, m->plan_no_values, &hp));
  if (total > 0) HL_TRY(sparse_adamw(m, total, kTableValue, hp));
  return HL_OK;
}

}  // namespace
}  // namespace hl

int hl_decoder_optimizer_step_sparse_rows(hl_decoder* m) {
  return hl_decoder_optimizer_step_policy(m, HL_MEMORY_UPDATE_SPARSE_ROWS);
}

int hl_decoder_optimizer_step_policy(hl_decoder* m, int policy) {
  HL_REQUIRE(m, "hl_decoder_optimizer_step_policy: null model");
  if (policy == HL_MEMORY_UPDATE_FROZEN) return HL_OK;  // no optimizer step at all (runtime.rs:2421-2423)
  HL_REQUIRE(m->has_opt, "hl_decoder: no optimizer configured (call hl_decoder_set_optimizer)");
  if (policy == HL_MEMORY_UPDATE_FULL) return hl_decoder_optimizer_step(m);
  HL_REQUIRE(m->has_memory, "hl_decoder_optimizer_step_policy: the model has no memory layers");
  const unsigned long long before = m->ctx->counters.launches;
  int rc;
  switch (policy) {
    case HL_MEMORY_UPDATE_MEMORY_ONLY: rc = hl::step_memory_only(m); break;
    case HL_MEMORY_UPDATE_SPARSE_ROWS: rc = hl::step_sparse_rows(m); break;
    case HL_MEMORY_UPDATE_DENSE_PLUS_SPARSE_VALUES: rc = hl::step_dense_plus_sparse_values(m); break;
    default: return hl::fail("hl_decoder_optimizer_step_policy: unknown policy " + std::to_string(policy));
  }
  m->launches_last_step += m->ctx->counters.launches - before;
  return rc;
}

int hl_decoder_memory_access_counts(hl_decoder* m, unsigned long long* counts_dev) {
  HL_REQUIRE(m && counts_dev, "hl_decoder_memory_access_counts: null argument");
  HL_REQUIRE(m->has_memory, "hl_decoder_memory_access_counts: the model has no memory layers");
  const long long per_layer = (long long)m->N * m->mem.top_k;
  for (int l = 0; l < m->cfg.n_layers; ++l)
    if (m->lo[l].is_memory)
      HL_TRY(hl_memory_access_count_rows_i64_u64(m->ctx, m->ma[l].idx, per_layer, m->mem.slots, counts_dev));
  return HL_OK;
}

int hl_decoder_set_smft_masks(hl_decoder* m, const unsigned char* value_mask_host, const unsigned char* left_mask_host,
                              const unsigned char* right_mask_host) {
  HL_REQUIRE(m, "hl_decoder_set_smft_masks: null model");
  HL_REQUIRE(m->has_memory, "hl_decoder_set_smft_masks: the model has no memory layers");
  if (!value_mask_host && !left_mask_host && !right_mask_host) { m->smft_on = false; return HL_OK; }
  HL_REQUIRE(value_mask_host && left_mask_host && right_mask_host, "hl_decoder_set_smft_masks: give all three masks or none");
  hl_ctx* ctx = m->ctx;
  HL_CUDA(cudaMemcpyAsync(m->smft_value_mask, value_mask_host, (size_t)m->mem.slots, cudaMemcpyHostToDevice, ctx->stream));
  HL_CUDA(cudaMemcpyAsync(m->smft_left_mask, left_mask_host, (size_t)m->side, cudaMemcpyHostToDevice, ctx->stream));
  HL_CUDA(cudaMemcpyAsync(m->smft_right_mask, right_mask_host, (size_t)m->side, cudaMemcpyHostToDevice, ctx->stream));
  HL_CUDA(cudaStreamSynchronize(ctx->stream));  // the host buffers may be freed on return
  m->smft_on = true;
  return HL_OK;
}

int hl_decoder_train_step_device(hl_decoder* m, const int64_t* tokens_dev, const int64_t* targets_dev) {
  HL_TRY(hl_decoder_forward_backward(m, tokens_dev, targets_dev));
  return hl_decoder_optimizer_step(m);
}

int hl_decoder_train_step(hl_decoder* m, const int64_t* tokens_host, const int64_t* targets_host, float* loss_host) {
  HL_REQUIRE(m && tokens_host && targets_host, "hl_decoder_train_step: null argument");
  hl_ctx* ctx = m->ctx;
  HL_CUDA(cudaMemcpyAsync(m->tokens, tokens_host, sizeof(int64_t) * m->N, cudaMemcpyHostToDevice, ctx->stream));
  HL_CUDA(cudaMemcpyAsync(m->targets, targets_host, sizeof(int64_t) * m->N, cudaMemcpyHostToDevice, ctx->stream));
  ctx->counters.h2d_bytes += 2 * sizeof(int64_t) * (size_t)m->N;
  HL_TRY(hl_decoder_forward_backward(m, m->tokens, m->targets));
  HL_TRY(hl_decoder_optimizer_step(m));
  HL_CUDA(cudaMemcpyAsync(m->loss_host, m->loss_dev, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  ctx->counters.d2h_bytes += sizeof(float);
  HL_TRY(hl_ctx_sync(ctx));
  if (loss_host) *loss_host = m->loss_host[0];
  return HL_OK;
}

namespace {
// Runs the forward pass over `sequences` rows of `time` tokens (both at most what the model was
// created for), restoring the configured sizes afterwards.
struct ScopedShape {
  hl_decoder* m;
  int batch, context, n;
  ScopedShape(hl_decoder* model, int sequences, int time) : m(model), batch(model->cfg.batch), context(model->cfg.context), n(model->N) {
    m->cfg.batch = sequences;
    m->cfg.context = time;
    m->N = sequences * time;
  }
  ~ScopedShape() {
    m->cfg.batch = batch;
    m->cfg.context = context;
    m->N = n;
  }
};
}  // namespace

int hl_decoder_eval_loss(hl_decoder* m, const int64_t* tokens_dev, const int64_t* targets_dev, int sequences,
                         float* loss_host) {
  HL_REQUIRE(m && tokens_dev && targets_dev && loss_host, "hl_decoder_eval_loss: null argument");
  HL_REQUIRE(sequences > 0 && sequences <= m->cfg.batch,
             "hl_decoder_eval_loss: sequences must be between 1 and the batch the model was created for");
  const size_t n = (size_t)sequences * m->cfg.context;
  HL_CUDA(cudaMemcpyAsync(m->tokens, tokens_dev, sizeof(int64_t) * n, cudaMemcpyDeviceToDevice, m->ctx->stream));
  HL_CUDA(cudaMemcpyAsync(m->targets, targets_dev, sizeof(int64_t) * n, cudaMemcpyDeviceToDevice, m->ctx->stream));
  {
    ScopedShape shape(m, sequences, m->cfg.context);
    if (m->cfg.precision == HL_PRECISION_AMP_BF16) HL_TRY(forward(m));
    else HL_TRY(forward_f32(m));
    HL_TRY(cross_entropy_impl(m->ctx, m->logits, m->cfg.vocab, m->targets, m->N, m->cfg.vocab, 1.0f, m->loss_dev, nullptr,
                              nullptr, HL_BF16, m->cfg.vocab));
  }
  return hl_memcpy_d2h(m->ctx, loss_host, m->loss_dev, sizeof(float));
}

int hl_decoder_next_token_logits(hl_decoder* m, const int64_t* window_dev, int window_len, float* logits_host) {
  HL_REQUIRE(m && window_dev && logits_host, "hl_decoder_next_token_logits: null argument");
  HL_REQUIRE(window_len >= 1, "next_token_logits requires at least one token");
  HL_REQUIRE(window_len <= m->cfg.context, "hl_decoder_next_token_logits: the window is longer than the model's context");
  HL_CUDA(cudaMemcpyAsync(m->tokens, window_dev, sizeof(int64_t) * window_len, cudaMemcpyDeviceToDevice, m->ctx->stream));
  {
    ScopedShape shape(m, 1, window_len);
    if (m->cfg.precision == HL_PRECISION_AMP_BF16) HL_TRY(forward(m));
    else HL_TRY(forward_f32(m));
  }
  return hl_memcpy_d2h(m->ctx, logits_host, m->logits + (size_t)(window_len - 1) * m->cfg.vocab, sizeof(float) * m->cfg.vocab);
}

int hl_decoder_loss(hl_decoder* m, float* loss_host) {
  HL_REQUIRE(m && loss_host, "hl_decoder_loss: null argument");
  return hl_memcpy_d2h(m->ctx, loss_host, m->loss_dev, sizeof(float));
}

unsigned long long hl_decoder_launches_last_step(hl_decoder* m) { return m ? m->launches_last_step : 0; }

int hl_decoder_comm_exposed_ms(hl_decoder* m, float* total_ms, int* waits) {
  HL_REQUIRE(m && total_ms, "hl_decoder_comm_exposed_ms: null argument");
  HL_CUDA(cudaStreamSynchronize(m->ctx->stream));
  float sum = 0.f;
  for (size_t i = 0; i < m->waits_recorded; ++i) {
    float ms = 0.f;
    HL_CUDA(cudaEventElapsedTime(&ms, m->wait_begin[i], m->wait_end[i]));
    sum += ms;
  }
  *total_ms = sum;
  if (waits) *waits = (int)m->waits_recorded;
  m->waits_recorded = 0;
  return HL_OK;
}

long long hl_ddp_bucket_count(long long arena_elems, long long bucket_elems) {
  if (arena_elems <= 0 || bucket_elems <= 0) return 0;
  return (arena_elems + bucket_elems - 1) / bucket_elems;
}

int hl_ddp_ready_buckets(long long arena_elems, long long bucket_elems, long long next_bucket, long long done_elems,
                         long long* starts, long long* counts, int capacity) {
  if (arena_elems <= 0 || bucket_elems <= 0 || next_bucket < 0 || !starts || !counts || capacity < 0) {
    hl::fail("hl_ddp_ready_buckets: invalid argument");
    return -1;
  }
  const long long total = hl_ddp_bucket_count(arena_elems, bucket_elems);
  int n = 0;
  for (long long b = next_bucket; b < total && n < capacity; ++b) {
    size_t start, end;
    hl::bucket_range((size_t)arena_elems, (size_t)bucket_elems, (size_t)b, &start, &end);
    if ((long long)end > done_elems) break;
    starts[n] = (long long)start;
    counts[n] = (long long)(end - start);
    ++n;
  }
  return n;
}

}  // extern "C"
