// Causal flash attention forward on tcgen05: S = Q·Kᵀ and O += P·V are tensor-memory
// accumulators, K/V tiles stream in by TMA, the online softmax runs in registers and P goes
// back to the tensor cores through swizzled shared memory.
//
// Replaces the reference's attention forward family — materialised [B,H,T,T] scores
// (src/tensor.rs:4459-4472, tensor_core.ptx:1785-2283) and the mma.sync flash forward that
// recomputes the same QK tile in every one of its hd/8 CTAs (tensor_core.ptx:2284-2981,
// heirloom-kernels/src/cuda.rs:5338-5359).  Saves the per-row log-sum-exp instead of
// row_max/row_denom.
//
// Layout: q, k, v are bf16 row-major [B*T, *] views with heads interleaved along the channel
// dimension (column h*hd + j, as src/tensor.rs:5156-5177), so they may live side by side in
// one fused [B*T, 3C] projection buffer.  One CTA owns 128 query rows of one (batch, head).
//
// Pipeline: key tiles of 64; two S buffers and the O accumulator in tensor memory and two P buffers in
// shared memory.  Four softmax warps (one per tensor-memory lane group, a thread per query row) work
// on tile j while the tensor cores run P·V of tile j-1 and Q·Kᵀ of tile j+1.  P is formed against a
// reference maximum that a row raises only when its maximum has grown by more than 2^8; the row then
// rescales its O in place (tensor-memory load, multiply, store) between two P·V products.  The CTA
// is sized (192 threads, 98 KB of shared memory, 256 tensor-memory columns) so that two of them share
// an SM and one's start-up and drain overlap the other's work.
#include "common.cuh"
#include "tc05.cuh"

namespace hl {
namespace {

constexpr int FA_BM = 128;   // query rows per CTA
constexpr int FA_BN = 64;    // keys per tile
constexpr int FA_KV_STAGES = 3;
constexpr int FA_P_BYTES = FA_BM * FA_BN * 2;   // 16 KB: 128 rows of 64 keys, one 128-byte line each
constexpr int FA_SOFTMAX_WARPS = 4;
constexpr int FA_THREADS = (FA_SOFTMAX_WARPS + 2) * 32;  // + TMA warp + MMA warp
constexpr int FA_TMEM_COLS = 256;  // S: 2 x 64 columns, O: head_dim columns (allocations are powers of two)

// Sizes that depend on the head dimension (64 or 128).  Operands wider than one 128-byte swizzle row are kept as
// blocks of 64 channels side by side: a Q block is [128 rows x 128 bytes], a K or V block [64 keys x 128 bytes].
template <int HD>
struct FaSizes {
  static_assert(HD == 64 || HD == 128, "head_dim 64 or 128");
  static constexpr int BLOCKS = HD / 64;
  static constexpr int Q_BLOCK = FA_BM * 128;            // 16 KB
  static constexpr int KV_BLOCK = FA_BN * 128;           // 8 KB
  static constexpr int Q_BYTES = BLOCKS * Q_BLOCK;
  static constexpr int KV_BYTES = BLOCKS * KV_BLOCK;
  static constexpr int SMEM_DATA = Q_BYTES + 2 * FA_KV_STAGES * KV_BYTES + 2 * FA_P_BYTES;  // 96 KB / 160 KB
  static constexpr int SMEM_BYTES = SMEM_DATA + 2048;    // barriers in front, alignment slack
  static constexpr int CTAS_PER_SM = HD == 64 ? 2 : 1;
  static_assert(CTAS_PER_SM * (SMEM_BYTES + 1024) <= 228 * 1024, "shared memory per SM");
  static_assert(2 * FA_BN + HD <= FA_TMEM_COLS, "tensor memory columns");
};

struct FaShared {
  uint64_t q_full;
  uint64_t k_full[FA_KV_STAGES], k_empty[FA_KV_STAGES];
  uint64_t v_full[FA_KV_STAGES], v_empty[FA_KV_STAGES];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(FaShared) + 1023 <= 2048, "front matter must fit the slack");

struct FaParams {
  int B, T, H;
  long long ld_out;
  __nv_bfloat16* out;
  float* lse;
  float scale_log2;  // softmax scale times log2(e)
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, FaSizes<HD>::CTAS_PER_SM)
flash_attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                           const FaParams p) {
  using Z = FaSizes<HD>;
  constexpr int FA_HD = HD;
  constexpr int FA_Q_BYTES = Z::Q_BYTES, FA_KV_BYTES = Z::KV_BYTES, FA_SMEM_DATA = Z::SMEM_DATA, FA_SMEM_BYTES = Z::SMEM_BYTES;
  extern __shared__ uint8_t fa_smem_raw[];
  const uintptr_t raw = reinterpret_cast<uintptr_t>(fa_smem_raw);
  uint8_t* tiles = reinterpret_cast<uint8_t*>((raw + sizeof(FaShared) + 1023) & ~uintptr_t(1023));
  FaShared* sh = reinterpret_cast<FaShared*>(fa_smem_raw);
  const bool layout_ok = (tiles + FA_SMEM_DATA) <= (fa_smem_raw + FA_SMEM_BYTES);
  uint8_t* sq = tiles;
  uint8_t* sk = sq + FA_Q_BYTES;
  uint8_t* sv = sk + FA_KV_STAGES * FA_KV_BYTES;
  uint8_t* sp = sv + FA_KV_STAGES * FA_KV_BYTES;  // two P buffers
  volatile int* abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.T + FA_BM - 1) / FA_BM;
  const int bh = blockIdx.x % (p.B * p.H);
  const int qi = nq - 1 - blockIdx.x / (p.B * p.H);  // heavy (late) query tiles are scheduled first
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qi * FA_BM;
  const int n_tiles = 2 * (qi + 1);  // key tiles of 64 up to and including the diagonal
  const int row_base = b * p.T;  // first row of this batch in the [B*T, *] views

  if (threadIdx.x == 0) {
    tc05::mbar_init(&sh->q_full, 1);
    for (int s = 0; s < FA_KV_STAGES; ++s) {
      tc05::mbar_init(&sh->k_full[s], 1);
      tc05::mbar_init(&sh->k_empty[s], 1);
      tc05::mbar_init(&sh->v_full[s], 1);
      tc05::mbar_init(&sh->v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc05::mbar_init(&sh->s_full[i], 1);
      tc05::mbar_init(&sh->p_full[i], FA_SOFTMAX_WARPS);
      tc05::mbar_init(&sh->o_full[i], 1);
    }
    sh->abort_flag = layout_ok ? 0 : 1;
    tc05::fence_barrier_init();
  }
  if (warp == FA_SOFTMAX_WARPS + 1) {
    tc05::tmem_alloc(&sh->tmem_base, FA_TMEM_COLS);
    tc05::tmem_relinquish();
  }
  tc05::tc_fence_before_sync();
  __syncthreads();
  tc05::tc_fence_after_sync();
  const uint32_t tmem_s0 = sh->tmem_base;         // S buffers at +0 and +64
  const uint32_t tmem_o0 = tmem_s0 + 2 * FA_BN;   // O at +128

  if (warp == FA_SOFTMAX_WARPS) {
    // -------------------------------------------------------------------------- TMA producer
    if (tc05::elect_one() && !*abort_flag) {
      tc05::tma_prefetch_desc(&map_q);
      tc05::tma_prefetch_desc(&map_k);
      tc05::tma_prefetch_desc(&map_v);
      tc05::mbar_arrive_expect_tx(&sh->q_full, FA_Q_BYTES);
#pragma unroll
      for (int blk = 0; blk < Z::BLOCKS; ++blk)
        tc05::tma_load_2d(sq + blk * Z::Q_BLOCK, &map_q, &sh->q_full, h * FA_HD + blk * 64, row_base + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % FA_KV_STAGES;
        const uint32_t ph = (uint32_t)(j / FA_KV_STAGES) & 1u;
        if (!tc05::mbar_wait(&sh->k_empty[s], ph ^ 1u, abort_flag)) break;
        tc05::mbar_arrive_expect_tx(&sh->k_full[s], FA_KV_BYTES);
#pragma unroll
        for (int blk = 0; blk < Z::BLOCKS; ++blk)
          tc05::tma_load_2d(sk + s * FA_KV_BYTES + blk * Z::KV_BLOCK, &map_k, &sh->k_full[s], h * FA_HD + blk * 64,
                            row_base + j * FA_BN);
        if (!tc05::mbar_wait(&sh->v_empty[s], ph ^ 1u, abort_flag)) break;
        tc05::mbar_arrive_expect_tx(&sh->v_full[s], FA_KV_BYTES);
#pragma unroll
        for (int blk = 0; blk < Z::BLOCKS; ++blk)
          tc05::tma_load_2d(sv + s * FA_KV_BYTES + blk * Z::KV_BLOCK, &map_v, &sh->v_full[s], h * FA_HD + blk * 64,
                            row_base + j * FA_BN);
      }
    }
  } else if (warp == FA_SOFTMAX_WARPS + 1) {
    // -------------------------------------------------------------------------- MMA issuer
    if (tc05::elect_one() && !*abort_flag) {
      constexpr uint32_t idesc_qk = tc05::instr_desc_bf16_f32(FA_BM, FA_BN, false, false);
      constexpr uint32_t idesc_pv = tc05::instr_desc_bf16_f32(FA_BM, FA_HD, false, true);
      const uint32_t aq = tc05::smem_u32(sq);
      auto issue_qk = [&](int j) -> bool {  // S[j & 1] = Q · K(j)ᵀ
        const int s = j % FA_KV_STAGES;
        if (!tc05::mbar_wait(&sh->k_full[s], (uint32_t)(j / FA_KV_STAGES) & 1u, abort_flag)) return false;
        tc05::tc_fence_after_sync();
        const uint32_t ak = tc05::smem_u32(sk + s * FA_KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_HD / 16; ++ks)  // 16 channels a step; four steps per 64-channel block
          tc05::umma_ss(tmem_s0 + (uint32_t)((j & 1) * FA_BN),
                        tc05::smem_desc_sw128(aq + (ks / 4) * Z::Q_BLOCK + (ks % 4) * 32, 16, 1024),
                        tc05::smem_desc_sw128(ak + (ks / 4) * Z::KV_BLOCK + (ks % 4) * 32, 16, 1024), idesc_qk,
                        ks > 0 ? 1u : 0u);
        tc05::umma_commit(&sh->k_empty[s]);
        tc05::umma_commit(&sh->s_full[j & 1]);
        return true;
      };
      bool ok = tc05::mbar_wait(&sh->q_full, 0, abort_flag);
      if (ok) ok = issue_qk(0);
      if (ok && n_tiles > 1) ok = issue_qk(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // P(j) is in shared memory, which also means S(j) has been read out of tensor memory
        if (!tc05::mbar_wait(&sh->p_full[j & 1], (uint32_t)(j >> 1) & 1u, abort_flag)) break;
        tc05::tc_fence_after_sync();
        const int s = j % FA_KV_STAGES;
        if (!tc05::mbar_wait(&sh->v_full[s], (uint32_t)(j / FA_KV_STAGES) & 1u, abort_flag)) break;
        tc05::tc_fence_after_sync();
        const uint32_t av = tc05::smem_u32(sv + s * FA_KV_BYTES);
        const uint32_t ap = tc05::smem_u32(sp + (j & 1) * FA_P_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          // A = P: [128 rows x 64 keys], K-major; B = V: rows are keys (MN-major), 16 keys per step
          const uint64_t da = tc05::smem_desc_sw128(ap + ks * 32, 16, 1024);
          const uint64_t db = tc05::smem_desc_sw128(av + ks * (16 * 128), Z::KV_BLOCK, 1024);  // channel blocks KV_BLOCK apart
          tc05::umma_ss(tmem_o0, da, db, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);  // O accumulates over the key tiles
        }
        tc05::umma_commit(&sh->v_empty[s]);
        tc05::umma_commit(&sh->o_full[j & 1]);
        if (j + 2 < n_tiles && !issue_qk(j + 2)) break;
      }
    }
  } else {
    // -------------------------------------------------------------------------- softmax warps
    const int r = warp * 32 + lane;     // query row within the tile == tensor-memory lane
    const int t = q0 + r;               // query position within the batch
    const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
    // O accumulates in tensor memory against a reference maximum m_ref that is only raised when a row's maximum has
    // grown by more than 2^8 since: P = 2^(s - m_ref) then stays below 256, which costs bf16 nothing (same relative
    // precision) and f32 sums nothing, and O is rescaled in place a few times per row instead of once per tile.
    constexpr float kRaise = 8.0f;
    float m_ref = -INFINITY;   // reference maximum, in log2 units
    float l_run = 0.f;         // row sum, scaled to m_ref
    bool ok = !*abort_flag;

    for (int j = 0; j < n_tiles && ok; ++j) {
      // P·V of tile j-2 has finished: its P buffer is free for this tile
      if (j >= 2) {
        if (!tc05::mbar_wait(&sh->o_full[j & 1], (uint32_t)((j - 2) >> 1) & 1u, abort_flag)) { ok = false; break; }
      }
      if (!tc05::mbar_wait(&sh->s_full[j & 1], (uint32_t)(j >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc05::tc_fence_after_sync();
      const bool diag = (j >= n_tiles - 2);  // the two tiles that hold keys q0 .. q0+127
      const int key0 = j * FA_BN;
      uint32_t sb[FA_BN];
      tc05::tmem_ld_32x32b_x32(tmem_s0 + (uint32_t)((j & 1) * FA_BN) + lane_sel, *reinterpret_cast<uint32_t(*)[32]>(&sb[0]));
      tc05::tmem_ld_32x32b_x32(tmem_s0 + (uint32_t)((j & 1) * FA_BN) + lane_sel + 32, *reinterpret_cast<uint32_t(*)[32]>(&sb[32]));
      tc05::tmem_ld_wait();
      // maximum of the raw scores (the scale is positive); masked entries become -inf
      float m_tile = -INFINITY;
      if (diag) {
#pragma unroll
        for (int i = 0; i < FA_BN; ++i)
          if (key0 + i > t) sb[i] = 0xff800000u;
      }
      {  // eight independent running maxima, so that the 64 comparisons are not one dependent chain
        float mx[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) mx[u] = __uint_as_float(sb[u]);
#pragma unroll
        for (int i = 8; i < FA_BN; ++i) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(sb[i]));
        m_tile = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
      }
      const float m_new = m_tile * p.scale_log2;  // finite in tile 0: key 0 is visible to every row
      const bool raise = m_new > m_ref + kRaise;  // always true in tile 0 (m_ref = -inf)
      if (j == 0) {
        m_ref = m_new;
      } else if (__any_sync(0xffffffffu, raise)) {
        // rows of this warp rescale their O in place; P·V of tile j-1 must have landed, and P·V of tile j is not
        // issued before this warp has handed over P(j)
        if (!tc05::mbar_wait(&sh->o_full[(j - 1) & 1], (uint32_t)((j - 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc05::tc_fence_after_sync();
        const float a = raise ? ex2_fast(m_ref - m_new) : 1.0f;
        if (raise) m_ref = m_new;
        l_run *= a;
#pragma unroll
        for (int hb = 0; hb < FA_HD / 32; ++hb) {
          uint32_t ob[32];
          tc05::tmem_ld_32x32b_x32(tmem_o0 + lane_sel + hb * 32, ob);
          tc05::tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; ++k) ob[k] = __float_as_uint(__uint_as_float(ob[k]) * a);
          tc05::tmem_st_32x32b_x32(tmem_o0 + lane_sel + hb * 32, ob);
        }
        tc05::tmem_st_wait();
      }
      const float neg_m = -m_ref;
      uint8_t* line = sp + (j & 1) * FA_P_BYTES + r * 128;
      float l_tile = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2_fast(fmaf(__uint_as_float(sb[q * 8 + 2 * e]), p.scale_log2, neg_m));
          const float p1 = ex2_fast(fmaf(__uint_as_float(sb[q * 8 + 2 * e + 1]), p.scale_log2, neg_m));
          l_tile += p0 + p1;
          w[e] = pack_bf16x2(p0, p1);
        }
        *reinterpret_cast<uint4*>(line + ((q ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_run += l_tile;
      tc05::fence_proxy_async_smem();
      tc05::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&sh->p_full[j & 1]);
    }
    if (ok) {  // the last P·V has landed
      ok = tc05::mbar_wait(&sh->o_full[(n_tiles - 1) & 1], (uint32_t)((n_tiles - 1) >> 1) & 1u, abort_flag);
      tc05::tc_fence_after_sync();
    }
    if (ok) {
      // O leaves through the Q tile's shared memory (every product that read Q has finished): a warp stages its 32
      // rows per 64-channel block (128-byte rows, 128-byte swizzle) and its lane 0 sends them with one TMA store, whole
      // 128-byte row segments instead of 16-byte stores that each touch 32 different lines.  Rows past T are clipped by
      // the tensor map.
      const float inv = 1.0f / l_run;
#pragma unroll
      for (int hb = 0; hb < FA_HD / 32; ++hb) {
        uint32_t ob[32];
        tc05::tmem_ld_32x32b_x32(tmem_o0 + lane_sel + hb * 32, ob);
        tc05::tmem_ld_wait();
        uint8_t* line = sq + (hb / 2) * Z::Q_BLOCK + r * 128;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(ob[i]) * inv, __uint_as_float(ob[i + 1]) * inv);
          o.y = pack_bf16x2(__uint_as_float(ob[i + 2]) * inv, __uint_as_float(ob[i + 3]) * inv);
          o.z = pack_bf16x2(__uint_as_float(ob[i + 4]) * inv, __uint_as_float(ob[i + 5]) * inv);
          o.w = pack_bf16x2(__uint_as_float(ob[i + 6]) * inv, __uint_as_float(ob[i + 7]) * inv);
          const int chunk = (hb & 1) * 4 + i / 8;  // 16-byte chunk of the 128-byte row
          *reinterpret_cast<uint4*>(line + ((chunk ^ (r & 7)) << 4)) = o;
        }
      }
      tc05::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int blk = 0; blk < Z::BLOCKS; ++blk)
          tc05::tma_store_3d(&map_o, sq + blk * Z::Q_BLOCK + warp * (32 * 128), h * FA_HD + blk * 64, q0 + warp * 32, b);
        tc05::tma_store_commit();
        tc05::tma_store_wait_all();
      }
    }
    if (ok && t < p.T) {
      // natural-log log-sum-exp of the scaled scores
      p.lse[((size_t)b * p.H + h) * p.T + t] = (m_ref + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  tc05::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    if (threadIdx.x == 0) atomicExch(p.status + (layout_ok ? ST_WAIT_EXPIRED : ST_BAD_ARGUMENT), 1);
  }
  if (warp == FA_SOFTMAX_WARPS + 1) {
    tc05::tc_fence_after_sync();
    tc05::tmem_dealloc(tmem_s0, FA_TMEM_COLS);
  }
}

}  // namespace

int flash_attention_forward_impl(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv, void* out,
                                 long long ld_out, float* lse, int batch, int time, int n_heads, int head_dim) {
  HL_REQUIRE(ctx && q && k && v && out && lse, "hl_flash_attention_forward: null argument");
  HL_REQUIRE(n_heads > 0, "hl_flash_attention_forward: causal_self_attention requires n_heads > 0");
  HL_REQUIRE(batch > 0 && time > 0, "hl_flash_attention_forward: batch and time must be positive");
  HL_REQUIRE(head_dim == 64 || head_dim == 128, "hl_flash_attention_forward: head_dim must be 64 or 128");
  HL_REQUIRE(ld_qkv % 8 == 0 && ld_out % 8 == 0 && ld_qkv >= (long long)n_heads * head_dim &&
                 ld_out >= (long long)n_heads * head_dim,
             "hl_flash_attention_forward: row strides must be multiples of 8 and cover all heads");
  HL_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
               reinterpret_cast<uintptr_t>(out)) & 15) == 0,
             "hl_flash_attention_forward: pointers must be 16-byte aligned");
  const uint64_t rows = (uint64_t)batch * time, cols = (uint64_t)n_heads * head_dim;
  CUtensorMap mq, mk, mv;
  int rc;
  // boxes of 64 channels (one 128-byte swizzle row); wider heads take several boxes per tile
  if ((rc = make_tensor_map_bf16_2d(&mq, q, cols, rows, (uint64_t)ld_qkv, 64, FA_BM)) != HL_OK) return rc;
  if ((rc = make_tensor_map_bf16_2d(&mk, k, cols, rows, (uint64_t)ld_qkv, 64, FA_BN)) != HL_OK) return rc;
  if ((rc = make_tensor_map_bf16_2d(&mv, v, cols, rows, (uint64_t)ld_qkv, 64, FA_BN)) != HL_OK) return rc;
  // the output as [batch][time][channels], so that a tile's rows past `time` are clipped; boxes of 64 channels by 32 rows
  CUtensorMap mo;
  {
    const uint64_t dims[3] = {(uint64_t)cols, (uint64_t)time, (uint64_t)batch};
    const uint64_t strides[2] = {(uint64_t)ld_out * 2, (uint64_t)time * (uint64_t)ld_out * 2};
    const uint32_t box[3] = {64, 32, 1};
    if ((rc = make_tensor_map(&mo, HL_BF16, 3, out, dims, strides, box, 128)) != HL_OK) return rc;
  }
  FaParams p{};
  p.B = batch; p.T = time; p.H = n_heads;
  p.ld_out = ld_out;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
  p.status = ctx->status_dev;
  const int nq = ceil_div(time, FA_BM);
  // causal algorithmic work: QK^T and PV over the lower triangle
  ProfileScope prof(ctx, HL_PROF_ATTENTION_FWD, 2.0 * batch * n_heads * (double)time * time * head_dim);
  if (head_dim == 64) {
    static bool configured = false;
    if (!configured) {
      HL_CUDA(cudaFuncSetAttribute(flash_attention_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSizes<64>::SMEM_BYTES));
      configured = true;
    }
    flash_attention_fwd_kernel<64><<<nq * batch * n_heads, FA_THREADS, FaSizes<64>::SMEM_BYTES, ctx->stream>>>(mq, mk, mv, mo, p);
  } else {
    static bool configured = false;
    if (!configured) {
      HL_CUDA(cudaFuncSetAttribute(flash_attention_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSizes<128>::SMEM_BYTES));
      configured = true;
    }
    flash_attention_fwd_kernel<128><<<nq * batch * n_heads, FA_THREADS, FaSizes<128>::SMEM_BYTES, ctx->stream>>>(mq, mk, mv, mo, p);
  }
  HL_LAUNCH_CHECK("flash_attention_fwd_kernel");
  count_launch(ctx);
  ctx->counters.attention_launches += 1;
  return HL_OK;
}

}  // namespace hl

extern "C" int hl_flash_attention_forward(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv,
                                          void* out, long long ld_out, float* lse, int batch, int time, int n_heads,
                                          int head_dim) {
  return hl::flash_attention_forward_impl(ctx, q, k, v, ld_qkv, out, ld_out, lse, batch, time, n_heads, head_dim);
}
