// Causal flash attention forward on tcgen05: S = Q·Kᵀ and O_tile = P·V are tensor-memory
// accumulators, K/V tiles stream in by TMA, the online softmax runs in registers (one thread
// per query row) and P goes back to the tensor cores through swizzled shared memory.
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
#include "common.cuh"
#include "tc05.cuh"

namespace hl {
namespace {

constexpr int FA_BM = 128;   // query rows per CTA
constexpr int FA_BN = 128;   // keys per tile
constexpr int FA_HD = 64;    // head dimension (one 128-byte swizzle row)
constexpr int FA_KV_STAGES = 2;
constexpr int FA_TILE_BYTES = 128 * FA_HD * 2;  // 16 KB
constexpr int FA_P_BYTES = FA_BM * FA_BN * 2;   // 32 KB
constexpr int FA_THREADS = 192;                 // warps 0-3 softmax, warp 4 TMA, warp 5 MMA
constexpr int FA_TMEM_COLS = 256;               // S: 128 columns, O tile: 64 columns
constexpr int FA_SMEM_DATA = FA_TILE_BYTES * (1 + 2 * FA_KV_STAGES) + FA_P_BYTES;  // 112 KB
constexpr int FA_SMEM_BYTES = FA_SMEM_DATA + 1024;  // barriers live in the alignment slack

struct FaBarriers {
  uint64_t q_full;
  uint64_t k_full[FA_KV_STAGES], k_empty[FA_KV_STAGES];
  uint64_t v_full[FA_KV_STAGES], v_empty[FA_KV_STAGES];
  uint64_t s_full, p_full, o_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct FaParams {
  int B, T, H;
  long long ld_out;
  __nv_bfloat16* out;
  float* lse;
  float scale_log2;  // softmax scale times log2(e)
  int* status;
};

__global__ void __launch_bounds__(FA_THREADS)
flash_attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const FaParams p) {
  extern __shared__ uint8_t fa_smem_raw[];
  // Tiles need 1024-byte alignment for the 128-byte swizzle; barriers use the bytes before them.
  const uintptr_t raw = reinterpret_cast<uintptr_t>(fa_smem_raw);
  uint8_t* tiles = reinterpret_cast<uint8_t*>((raw + sizeof(FaBarriers) + 1023) & ~uintptr_t(1023));
  FaBarriers* bars = reinterpret_cast<FaBarriers*>(fa_smem_raw);
  const bool layout_ok = (tiles + FA_SMEM_DATA) <= (fa_smem_raw + FA_SMEM_BYTES);
  uint8_t* sq = tiles;
  uint8_t* sk = sq + FA_TILE_BYTES;
  uint8_t* sv = sk + FA_KV_STAGES * FA_TILE_BYTES;
  uint8_t* sp = sv + FA_KV_STAGES * FA_TILE_BYTES;
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.T + FA_BM - 1) / FA_BM;
  const int bh = blockIdx.x % (p.B * p.H);
  const int qi = nq - 1 - blockIdx.x / (p.B * p.H);  // heavy (late) query tiles are scheduled first
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qi * FA_BM;
  const int n_tiles = qi + 1;
  const int row_base = b * p.T;  // first row of this batch in the [B*T, *] views

  if (threadIdx.x == 0) {
    tc05::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < FA_KV_STAGES; ++s) {
      tc05::mbar_init(&bars->k_full[s], 1);
      tc05::mbar_init(&bars->k_empty[s], 1);
      tc05::mbar_init(&bars->v_full[s], 1);
      tc05::mbar_init(&bars->v_empty[s], 1);
    }
    tc05::mbar_init(&bars->s_full, 1);
    tc05::mbar_init(&bars->p_full, 4);
    tc05::mbar_init(&bars->o_full, 1);
    bars->abort_flag = layout_ok ? 0 : 1;
    tc05::fence_barrier_init();
  }
  if (warp == 5) {
    tc05::tmem_alloc(&bars->tmem_base, FA_TMEM_COLS);
    tc05::tmem_relinquish();
  }
  tc05::tc_fence_before_sync();
  __syncthreads();
  tc05::tc_fence_after_sync();
  const uint32_t tmem_s = bars->tmem_base;
  const uint32_t tmem_o = tmem_s + FA_BN;

  if (warp == 4) {
    // -------------------------------------------------------------------------- TMA producer
    if (tc05::elect_one() && !*abort_flag) {
      tc05::tma_prefetch_desc(&map_q);
      tc05::tma_prefetch_desc(&map_k);
      tc05::tma_prefetch_desc(&map_v);
      tc05::mbar_arrive_expect_tx(&bars->q_full, FA_TILE_BYTES);
      tc05::tma_load_2d(sq, &map_q, &bars->q_full, h * FA_HD, row_base + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % FA_KV_STAGES;
        const uint32_t ph = (uint32_t)(j / FA_KV_STAGES) & 1u;
        if (!tc05::mbar_wait(&bars->k_empty[s], ph ^ 1u, abort_flag)) break;
        tc05::mbar_arrive_expect_tx(&bars->k_full[s], FA_TILE_BYTES);
        tc05::tma_load_2d(sk + s * FA_TILE_BYTES, &map_k, &bars->k_full[s], h * FA_HD, row_base + j * FA_BN);
        if (!tc05::mbar_wait(&bars->v_empty[s], ph ^ 1u, abort_flag)) break;
        tc05::mbar_arrive_expect_tx(&bars->v_full[s], FA_TILE_BYTES);
        tc05::tma_load_2d(sv + s * FA_TILE_BYTES, &map_v, &bars->v_full[s], h * FA_HD, row_base + j * FA_BN);
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------------------- MMA issuer
    if (tc05::elect_one() && !*abort_flag) {
      constexpr uint32_t idesc_qk = tc05::instr_desc_bf16_f32(FA_BM, FA_BN, false, false);
      constexpr uint32_t idesc_pv = tc05::instr_desc_bf16_f32(FA_BM, FA_HD, false, true);
      const uint32_t aq = tc05::smem_u32(sq), ap = tc05::smem_u32(sp);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % FA_KV_STAGES;
        if (!tc05::mbar_wait(&bars->k_full[s], (uint32_t)(j / FA_KV_STAGES) & 1u, abort_flag)) return false;
        tc05::tc_fence_after_sync();
        const uint32_t ak = tc05::smem_u32(sk + s * FA_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_HD / 16; ++ks)
          tc05::umma_ss(tmem_s, tc05::smem_desc_sw128(aq + ks * 32, 16, 1024),
                        tc05::smem_desc_sw128(ak + ks * 32, 16, 1024), idesc_qk, ks > 0 ? 1u : 0u);
        tc05::umma_commit(&bars->k_empty[s]);
        tc05::umma_commit(&bars->s_full);
        return true;
      };
      bool ok = tc05::mbar_wait(&bars->q_full, 0, abort_flag);
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // P(j) is in shared memory and S(j) has been read out: S may be overwritten.
        if (!tc05::mbar_wait(&bars->p_full, (uint32_t)j & 1u, abort_flag)) break;
        tc05::tc_fence_after_sync();
        if (j + 1 < n_tiles && !issue_qk(j + 1)) break;
        const int s = j % FA_KV_STAGES;
        if (!tc05::mbar_wait(&bars->v_full[s], (uint32_t)(j / FA_KV_STAGES) & 1u, abort_flag)) break;
        tc05::tc_fence_after_sync();
        const uint32_t av = tc05::smem_u32(sv + s * FA_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          // A = P: two 64-key blocks of [128 rows x 128 B]; B = V rows are keys (MN-major).
          const uint64_t da = tc05::smem_desc_sw128(ap + (ks / 4) * (FA_BM * 128) + (ks % 4) * 32, 16, 1024);
          const uint64_t db = tc05::smem_desc_sw128(av + ks * (16 * 128), FA_BN * 128, 1024);
          tc05::umma_ss(tmem_o, da, db, idesc_pv, ks > 0 ? 1u : 0u);
        }
        tc05::umma_commit(&bars->v_empty[s]);
        tc05::umma_commit(&bars->o_full);
      }
    }
  } else {
    // -------------------------------------------------------------------------- softmax warps
    const int r = warp * 32 + lane;            // query row within the tile == tensor-memory lane
    const int t = q0 + r;                      // query position within the batch
    const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
    float o_acc[FA_HD];
#pragma unroll
    for (int i = 0; i < FA_HD; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = !*abort_flag;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!tc05::mbar_wait(&bars->s_full, (uint32_t)j & 1u, abort_flag)) { ok = false; break; }
      tc05::tc_fence_after_sync();
      const bool diag = (j == n_tiles - 1);
      const int key0 = j * FA_BN;
      // pass 1: row maximum
      float m_tile = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < FA_BN / 32; ++c) {
        uint32_t sb[32];
        tc05::tmem_ld_32x32b_x32(tmem_s + lane_sel + c * 32, sb);
        tc05::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(sb[i]) * p.scale_log2;
          if (diag && key0 + c * 32 + i > t) s = -INFINITY;
          m_tile = fmaxf(m_tile, s);
        }
      }
      const float m_new = fmaxf(m_run, m_tile);
      const float alpha = exp2f(m_run - m_new);  // m_run = -inf on the first tile gives 0
      // pass 2: probabilities, row sum, P -> shared memory (K-major, 128-byte swizzle)
      float l_tile = 0.f;
#pragma unroll 1
      for (int c = 0; c < FA_BN / 32; ++c) {
        uint32_t sb[32];
        tc05::tmem_ld_32x32b_x32(tmem_s + lane_sel + c * 32, sb);
        tc05::tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(sb[i]) * p.scale_log2, s1 = __uint_as_float(sb[i + 1]) * p.scale_log2;
          if (diag && key0 + c * 32 + i > t) s0 = -INFINITY;
          if (diag && key0 + c * 32 + i + 1 > t) s1 = -INFINITY;
          const float p0 = exp2f(s0 - m_new), p1 = exp2f(s1 - m_new);
          l_tile += p0 + p1;
          packed[i / 2] = pack_bf16x2(p0, p1);
        }
        // 32 keys = four 16-byte chunks of this row's 128-byte line in key block c/2
        uint8_t* line = sp + (c / 2) * (FA_BM * 128) + r * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (c % 2) * 4 + q;
          *reinterpret_cast<uint4*>(line + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
        }
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      // hand P to the tensor cores
      tc05::fence_proxy_async_smem();
      tc05::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&bars->p_full);
      // fold O_tile = P·V into the running output
      if (!tc05::mbar_wait(&bars->o_full, (uint32_t)j & 1u, abort_flag)) { ok = false; break; }
      tc05::tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < FA_HD / 32; ++c) {
        uint32_t ob[32];
        tc05::tmem_ld_32x32b_x32(tmem_o + lane_sel + c * 32, ob);
        tc05::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(ob[i]);
      }
    }
    if (ok && t < p.T) {
      const float inv = 1.0f / l_run;
      __nv_bfloat16* dst = p.out + (size_t)(row_base + t) * p.ld_out + (size_t)h * FA_HD;
#pragma unroll
      for (int i = 0; i < FA_HD; i += 8) {
        uint4 o;
        o.x = pack_bf16x2(o_acc[i] * inv, o_acc[i + 1] * inv);
        o.y = pack_bf16x2(o_acc[i + 2] * inv, o_acc[i + 3] * inv);
        o.z = pack_bf16x2(o_acc[i + 4] * inv, o_acc[i + 5] * inv);
        o.w = pack_bf16x2(o_acc[i + 6] * inv, o_acc[i + 7] * inv);
        *reinterpret_cast<uint4*>(dst + i) = o;
      }
      // natural-log log-sum-exp of the scaled scores
      p.lse[((size_t)b * p.H + h) * p.T + t] = (m_run + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  tc05::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    if (threadIdx.x == 0) atomicExch(p.status + (layout_ok ? ST_WAIT_EXPIRED : ST_BAD_ARGUMENT), 1);
  }
  if (warp == 5) {
    tc05::tc_fence_after_sync();
    tc05::tmem_dealloc(tmem_s, FA_TMEM_COLS);
  }
}

}  // namespace

int flash_attention_forward_impl(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv, void* out,
                                 long long ld_out, float* lse, int batch, int time, int n_heads, int head_dim) {
  HL_REQUIRE(ctx && q && k && v && out && lse, "hl_flash_attention_forward: null argument");
  HL_REQUIRE(n_heads > 0, "hl_flash_attention_forward: causal_self_attention requires n_heads > 0");
  HL_REQUIRE(batch > 0 && time > 0, "hl_flash_attention_forward: batch and time must be positive");
  HL_REQUIRE(head_dim == FA_HD, "hl_flash_attention_forward: head_dim must be 64");
  HL_REQUIRE(ld_qkv % 8 == 0 && ld_out % 8 == 0 && ld_qkv >= (long long)n_heads * head_dim &&
                 ld_out >= (long long)n_heads * head_dim,
             "hl_flash_attention_forward: row strides must be multiples of 8 and cover all heads");
  HL_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
               reinterpret_cast<uintptr_t>(out)) & 15) == 0,
             "hl_flash_attention_forward: pointers must be 16-byte aligned");
  const uint64_t rows = (uint64_t)batch * time, cols = (uint64_t)n_heads * head_dim;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_tensor_map_bf16_2d(&mq, q, cols, rows, (uint64_t)ld_qkv, FA_HD, FA_BM)) != HL_OK) return rc;
  if ((rc = make_tensor_map_bf16_2d(&mk, k, cols, rows, (uint64_t)ld_qkv, FA_HD, FA_BN)) != HL_OK) return rc;
  if ((rc = make_tensor_map_bf16_2d(&mv, v, cols, rows, (uint64_t)ld_qkv, FA_HD, FA_BN)) != HL_OK) return rc;
  FaParams p{};
  p.B = batch; p.T = time; p.H = n_heads;
  p.ld_out = ld_out;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
  p.status = ctx->status_dev;
  static bool configured = false;
  if (!configured) {
    HL_CUDA(cudaFuncSetAttribute(flash_attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM_BYTES));
    configured = true;
  }
  const int nq = ceil_div(time, FA_BM);
  // causal algorithmic work: QK^T and PV over the lower triangle
  ProfileScope prof(ctx, HL_PROF_ATTENTION_FWD, 2.0 * batch * n_heads * (double)time * time * head_dim);
  flash_attention_fwd_kernel<<<nq * batch * n_heads, FA_THREADS, FA_SMEM_BYTES, ctx->stream>>>(mq, mk, mv, p);
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
