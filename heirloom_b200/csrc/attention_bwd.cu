// Causal flash attention backward on tcgen05.  A work item is 128 keys of one (batch, head) and
// walks the query tiles at or below the diagonal; one persistent CTA per SM takes items round-robin
// (longest walks first) and starts the next item's loads and first products while the current one
// drains.  Per query tile five tensor-core products
// run against tensor memory:
//     S  = Q·Kᵀ          dP = dO·Vᵀ                      (recomputed scores, f32)
//     dV += Pᵀ·dO        dK += dSᵀ·Q        dQ_tile = dS·K
// P = exp(S·scale − lse) and dS = P∘(dP − D)·scale are formed in registers by eight warps (two
// per tensor-memory lane group, each taking half of the key columns) and handed back through
// swizzled shared memory as bf16 operands.  dK and dV stay in tensor memory for the whole
// walk; dQ tiles are staged in shared memory and added into an f32 accumulator by TMA reductions.
//
// Replaces the reference's recompute-based backward with scalar f32 atomics
// (tensor_core.ptx:3111-4407, heirloom-kernels/src/cuda.rs:9256-9294) and, for the values it
// computes, follows src/tensor/autograd.rs:1626-1914 (bf16 operands, f32 accumulation).
#include <type_traits>

#include "common.cuh"
#include "tc05.cuh"

namespace hl {
namespace {

constexpr int FB_BM = 128;  // queries per tile
constexpr int FB_BN = 128;  // keys per work item
constexpr int FB_BLOCK = 128 * 128;  // one 64-channel block of a 128-row operand tile: 16 KB
constexpr int FB_PS_BYTES = FB_BM * FB_BN * 2;  // 32 KB
constexpr int FB_SOFTMAX_WARPS = 8;
constexpr int FB_THREADS = (FB_SOFTMAX_WARPS + 2) * 32;  // + TMA warp + MMA warp
constexpr int FB_TMEM_COLS = 512;
constexpr int FB_DQ_BYTES = FB_BM * 64 * 4;     // 32 KB: 64 columns of a dQ tile in f32, staged for the TMA reduction
constexpr int FB_MAX_STAGES = 2;

// Sizes that depend on the head dimension.  A head of 128 channels is worked on as two halves of 64: S and dP use the
// whole head (their operand tiles are two 64-channel blocks side by side), while dV, dK and dQ of a work item cover
// one 64-channel block, so that the tensor-memory budget (S 128 + dP 128 + dV 64 + dK 64 + dQ 2 x 64 columns) is the
// same for both sizes; the two halves are separate work items.  The wider tiles leave room for one K/V buffer and
// one Q/dO stage only.
template <int HD>
struct FbSizes {
  static_assert(HD == 64 || HD == 128, "head_dim 64 or 128");
  static constexpr int BLOCKS = HD / 64;
  static constexpr int TILE_BYTES = BLOCKS * FB_BLOCK;  // 16 KB / 32 KB
  static constexpr int KV_BUFFERS = HD == 64 ? 2 : 1;
  static constexpr int Q_STAGES = HD == 64 ? 2 : 1;
  static constexpr int SMEM_DATA = TILE_BYTES * (2 * KV_BUFFERS + 2 * Q_STAGES) + 2 * FB_PS_BYTES + FB_DQ_BYTES;  // 224 KB
  static constexpr int SMEM_BYTES = SMEM_DATA + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct FbBarriers {
  uint64_t kv_full[FB_MAX_STAGES], kv_empty[FB_MAX_STAGES];
  uint64_t q_full[FB_MAX_STAGES], q_empty[FB_MAX_STAGES];
  uint64_t sdp_full, sdp_free, p_full, dq_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct FbParams {
  int B, T, H;
  int blocks;          // 64-channel blocks per head: 1 or 2
  const float* lse;    // [B,H,T]
  const float* delta;  // [B,H,T] rowsum(dO * O)
  float* dq_accum;     // f32 [B*T, H*hd], zeroed by the caller
  long long ld_dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long ld_dkv;
  float scale, scale_log2;
  int* status;
};

// A CTA's place in its sequence of query tiles: work item `item` (one key tile of one batch and
// head; items with the longest walks come first), query tile `it` of its walk.  Every warp role
// advances an identical copy.
struct FbCursor {
  int item;      // global work item, -1 when the sequence is over
  int local;     // how many items this CTA has started before this one
  int it;        // query tile within the item's walk
  int n_tiles;   // length of the walk
  int kj, b, h;  // key tile, batch, head
  int cb;        // which 64-channel block of the head this item's dV, dK and dQ cover
  __device__ __forceinline__ bool valid() const { return item >= 0; }
};
// The CTA's `local`-th item.  Items are sorted by decreasing walk length; rounds alternate direction
// (CTA 0 takes the longest item of even rounds and the shortest of odd ones), which evens out the
// per-CTA totals of a static assignment.
__device__ __forceinline__ void fb_load_item(FbCursor& c, int local, const FbParams& p) {
  const int nq = (p.T + FB_BM - 1) / FB_BM;
  const int per_kj = p.B * p.H * p.blocks;
  const int total = nq * per_kj;
  const int grid = (int)gridDim.x, cta = (int)blockIdx.x;
  const int item = local * grid + ((local & 1) ? grid - 1 - cta : cta);
  if (item >= total) { c.item = -1; return; }
  const int rest = item % per_kj;
  const int bh = rest / p.blocks;
  c.item = item;
  c.local = local;
  c.it = 0;
  c.kj = item / per_kj;
  c.cb = rest % p.blocks;
  c.b = bh / p.H;
  c.h = bh % p.H;
  c.n_tiles = nq - c.kj;  // query tiles kj .. nq-1
}
__device__ __forceinline__ FbCursor fb_next(const FbCursor& c, const FbParams& p) {
  FbCursor n = c;
  if (c.it + 1 < c.n_tiles) { n.it = c.it + 1; return n; }
  fb_load_item(n, c.local + 1, p);
  return n;
}

template <int HD>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_attention_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                           const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ CUtensorMap map_dk,
                           const __grid_constant__ CUtensorMap map_dv, const FbParams p) {
  using Z = FbSizes<HD>;
  constexpr int FB_HD = HD;
  constexpr int FB_TILE_BYTES = Z::TILE_BYTES, FB_KV_BUFFERS = Z::KV_BUFFERS, FB_Q_STAGES = Z::Q_STAGES;
  constexpr int FB_SMEM_DATA = Z::SMEM_DATA, FB_SMEM_BYTES = Z::SMEM_BYTES;
  extern __shared__ uint8_t fb_smem_raw[];
  const uintptr_t raw = reinterpret_cast<uintptr_t>(fb_smem_raw);
  uint8_t* tiles = reinterpret_cast<uint8_t*>((raw + sizeof(FbBarriers) + 1023) & ~uintptr_t(1023));
  FbBarriers* bars = reinterpret_cast<FbBarriers*>(fb_smem_raw);
  const bool layout_ok = (tiles + FB_SMEM_DATA) <= (fb_smem_raw + FB_SMEM_BYTES);
  uint8_t* sk = tiles;                                 // [buffer] K tiles
  uint8_t* sv = sk + FB_KV_BUFFERS * FB_TILE_BYTES;    // [buffer] V tiles
  uint8_t* sq = sv + FB_KV_BUFFERS * FB_TILE_BYTES;    // [stage] Q tiles
  uint8_t* sdo = sq + FB_Q_STAGES * FB_TILE_BYTES;     // [stage] dO tiles
  uint8_t* sp = sdo + FB_Q_STAGES * FB_TILE_BYTES;     // P  (bf16, [query][key], two 64-key blocks)
  uint8_t* sds = sp + FB_PS_BYTES;                     // dS (same layout)
  uint8_t* sdq = sds + FB_PS_BYTES;                    // dQ tile, f32: two blocks of [query][32 columns], 128-byte swizzle
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < FB_KV_BUFFERS; ++s) {
      tc05::mbar_init(&bars->kv_full[s], 1);
      tc05::mbar_init(&bars->kv_empty[s], 1);
    }
    for (int s = 0; s < FB_Q_STAGES; ++s) {
      tc05::mbar_init(&bars->q_full[s], 1);
      tc05::mbar_init(&bars->q_empty[s], 1);
    }
    tc05::mbar_init(&bars->sdp_full, 1);
    tc05::mbar_init(&bars->sdp_free, FB_SOFTMAX_WARPS);
    tc05::mbar_init(&bars->p_full, FB_SOFTMAX_WARPS);
    tc05::mbar_init(&bars->dq_full, 1);
    bars->abort_flag = layout_ok ? 0 : 1;
    tc05::fence_barrier_init();
  }
  if (warp == FB_SOFTMAX_WARPS + 1) {
    tc05::tmem_alloc(&bars->tmem_base, FB_TMEM_COLS);
    tc05::tmem_relinquish();
  }
  tc05::tc_fence_before_sync();
  __syncthreads();
  tc05::tc_fence_after_sync();
  const uint32_t tmem_s = bars->tmem_base;  // 128 columns
  const uint32_t tmem_dp = tmem_s + 128;    // 128 columns
  const uint32_t tmem_dv = tmem_s + 256;    // 64 columns (one channel block of the head)
  const uint32_t tmem_dk = tmem_s + 320;    // 64 columns
  const uint32_t tmem_dq = tmem_s + 384;    // two buffers of 64 columns, alternating by query tile

  FbCursor first;
  fb_load_item(first, 0, p);

  if (warp == FB_SOFTMAX_WARPS) {
    // -------------------------------------------------------------------------- TMA producer
    // Runs ahead of the other roles: the next item's K and V go into the other buffer pair while the
    // current item is still being worked on.
    if (tc05::elect_one() && !*abort_flag) {
      tc05::tma_prefetch_desc(&map_q);
      tc05::tma_prefetch_desc(&map_k);
      tc05::tma_prefetch_desc(&map_v);
      tc05::tma_prefetch_desc(&map_do);
      int g = 0;  // query tiles loaded so far
      for (FbCursor c = first; c.valid(); c = fb_next(c, p), ++g) {
        const int row_base = c.b * p.T;
        if (c.it == 0) {
          const int kb = c.local % FB_KV_BUFFERS;
          if (!tc05::mbar_wait(&bars->kv_empty[kb], ((uint32_t)(c.local / FB_KV_BUFFERS) & 1u) ^ 1u, abort_flag)) break;
          tc05::mbar_arrive_expect_tx(&bars->kv_full[kb], 2 * FB_TILE_BYTES);
#pragma unroll
          for (int blk = 0; blk < Z::BLOCKS; ++blk) {
            tc05::tma_load_2d(sk + kb * FB_TILE_BYTES + blk * FB_BLOCK, &map_k, &bars->kv_full[kb], c.h * FB_HD + blk * 64,
                              row_base + c.kj * FB_BN);
            tc05::tma_load_2d(sv + kb * FB_TILE_BYTES + blk * FB_BLOCK, &map_v, &bars->kv_full[kb], c.h * FB_HD + blk * 64,
                              row_base + c.kj * FB_BN);
          }
        }
        const int s = g % FB_Q_STAGES;
        const int qrow = row_base + (c.kj + c.it) * FB_BM;
        // the stage frees only when the tile two back has been consumed: have L2 fetch the tile in the meantime
#pragma unroll
        for (int blk = 0; blk < Z::BLOCKS; ++blk) {
          tc05::tma_prefetch_l2_2d(&map_q, c.h * FB_HD + blk * 64, qrow);
          tc05::tma_prefetch_l2_2d(&map_do, c.h * FB_HD + blk * 64, qrow);
        }
        if (!tc05::mbar_wait(&bars->q_empty[s], ((uint32_t)(g / FB_Q_STAGES) & 1u) ^ 1u, abort_flag)) break;
        tc05::mbar_arrive_expect_tx(&bars->q_full[s], 2 * FB_TILE_BYTES);
#pragma unroll
        for (int blk = 0; blk < Z::BLOCKS; ++blk) {
          tc05::tma_load_2d(sq + s * FB_TILE_BYTES + blk * FB_BLOCK, &map_q, &bars->q_full[s], c.h * FB_HD + blk * 64, qrow);
          tc05::tma_load_2d(sdo + s * FB_TILE_BYTES + blk * FB_BLOCK, &map_do, &bars->q_full[s], c.h * FB_HD + blk * 64, qrow);
        }
      }
    }
  } else if (warp == FB_SOFTMAX_WARPS + 1) {
    // -------------------------------------------------------------------------- MMA issuer
    if (tc05::elect_one() && !*abort_flag) {
      constexpr uint32_t idesc_sdp = tc05::instr_desc_bf16_f32(128, 128, false, false);
      constexpr uint32_t idesc_dkv = tc05::instr_desc_bf16_f32(128, 64, true, true);   // one channel block of dV / dK
      constexpr uint32_t idesc_dq = tc05::instr_desc_bf16_f32(128, 64, false, true);
      const uint32_t ap = tc05::smem_u32(sp), ads = tc05::smem_u32(sds);
      // S = Q·Kᵀ and dP = dO·Vᵀ of query tile number `g` (counted over the whole sequence)
      auto issue_scores = [&](const FbCursor& c, int g) -> bool {
        const int kb = c.local % FB_KV_BUFFERS;
        if (c.it == 0) {
          if (!tc05::mbar_wait(&bars->kv_full[kb], (uint32_t)(c.local / FB_KV_BUFFERS) & 1u, abort_flag)) return false;
        }
        const int s = g % FB_Q_STAGES;
        if (!tc05::mbar_wait(&bars->q_full[s], (uint32_t)(g / FB_Q_STAGES) & 1u, abort_flag)) return false;
        tc05::tc_fence_after_sync();
        const uint32_t ak = tc05::smem_u32(sk + kb * FB_TILE_BYTES), av = tc05::smem_u32(sv + kb * FB_TILE_BYTES);
        const uint32_t aq = tc05::smem_u32(sq + s * FB_TILE_BYTES), ado = tc05::smem_u32(sdo + s * FB_TILE_BYTES);
        // A descriptor's low bits are the operand's address in 16-byte units, so the steps along a tile are plain
        // additions to the first step's descriptor (no field overflows: shared memory ends below 256 KB).
        const uint64_t dq0 = tc05::smem_desc_sw128(aq, 16, 1024), dk0 = tc05::smem_desc_sw128(ak, 16, 1024);
        const uint64_t ddo0 = tc05::smem_desc_sw128(ado, 16, 1024), dv0 = tc05::smem_desc_sw128(av, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < FB_HD / 16; ++ks) {  // the whole head: four 16-channel steps per 64-channel block
          const uint64_t step = (uint64_t)((ks / 4) * (FB_BLOCK >> 4) + (ks % 4) * 2);
          tc05::umma_ss(tmem_s, dq0 + step, dk0 + step, idesc_sdp, ks > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < FB_HD / 16; ++ks) {
          const uint64_t step = (uint64_t)((ks / 4) * (FB_BLOCK >> 4) + (ks % 4) * 2);
          tc05::umma_ss(tmem_dp, ddo0 + step, dv0 + step, idesc_sdp, ks > 0 ? 1u : 0u);
        }
        tc05::umma_commit(&bars->sdp_full);
        return true;
      };
      FbCursor c = first;
      bool ok = c.valid() && issue_scores(c, 0);
      for (int g = 0; ok && c.valid(); ++g) {
        // S/dP of the next query tile (of this item or of the next one) are issued as soon as this
        // tile's have been read out, so the softmax warps find them ready when they come back
        const FbCursor n = fb_next(c, p);
        if (FB_Q_STAGES > 1 && n.valid()) {
          if (!tc05::mbar_wait(&bars->sdp_free, (uint32_t)g & 1u, abort_flag)) break;
          tc05::tc_fence_after_sync();
          if (!issue_scores(n, g + 1)) break;
        }
        if (!tc05::mbar_wait(&bars->p_full, (uint32_t)g & 1u, abort_flag)) break;
        tc05::tc_fence_after_sync();
        const int s = g % FB_Q_STAGES;
        const int kb = c.local % FB_KV_BUFFERS;
        // dV, dK and dQ of this item cover channel block c.cb of the head
        const uint32_t ak = tc05::smem_u32(sk + kb * FB_TILE_BYTES) + (uint32_t)(c.cb * FB_BLOCK);
        const uint32_t aq = tc05::smem_u32(sq + s * FB_TILE_BYTES) + (uint32_t)(c.cb * FB_BLOCK);
        const uint32_t ado = tc05::smem_u32(sdo + s * FB_TILE_BYTES) + (uint32_t)(c.cb * FB_BLOCK);
        const uint64_t a_pt0 = tc05::smem_desc_sw128(ap, FB_BM * 128, 1024);    // P^T  (keys x queries)
        const uint64_t a_dst0 = tc05::smem_desc_sw128(ads, FB_BM * 128, 1024);  // dS^T
        const uint64_t b_do0 = tc05::smem_desc_sw128(ado, FB_BM * 128, 1024);
        const uint64_t b_q0 = tc05::smem_desc_sw128(aq, FB_BM * 128, 1024);
#pragma unroll
        for (int ks = 0; ks < FB_BM / 16; ++ks) {
          // contraction over the 128 queries of this tile: 16 query rows = 2048 bytes = 128 address units per step
          const uint64_t step = (uint64_t)(ks * 128);
          const uint32_t acc = (c.it > 0 || ks > 0) ? 1u : 0u;  // a new item starts its dV/dK from zero
          tc05::umma_ss(tmem_dv, a_pt0 + step, b_do0 + step, idesc_dkv, acc);
          tc05::umma_ss(tmem_dk, a_dst0 + step, b_q0 + step, idesc_dkv, acc);
        }
        const uint64_t a_ds0 = tc05::smem_desc_sw128(ads, 16, 1024);
        const uint64_t b_k0 = tc05::smem_desc_sw128(ak, FB_BN * 128, 1024);
#pragma unroll
        for (int ks = 0; ks < FB_BN / 16; ++ks) {
          // dQ_tile = dS·K: contraction over the 128 keys; dS is K-major in two 64-key blocks
          const uint64_t a_step = (uint64_t)((ks / 4) * ((FB_BM * 128) >> 4) + (ks % 4) * 2);
          tc05::umma_ss(tmem_dq + (uint32_t)((g & 1) * 64), a_ds0 + a_step, b_k0 + (uint64_t)(ks * 128), idesc_dq, ks > 0 ? 1u : 0u);
        }
        tc05::umma_commit(&bars->q_empty[s]);
        if (c.it == c.n_tiles - 1) tc05::umma_commit(&bars->kv_empty[kb]);  // the item's K and V are no longer read
        tc05::umma_commit(&bars->dq_full);
        if (FB_Q_STAGES == 1 && n.valid()) {
          // one Q/dO stage: the next tile's loads could only start once this tile's products were committed, so its
          // scores are issued after them (S and dP were read out before P and dS were handed over)
          if (!tc05::mbar_wait(&bars->sdp_free, (uint32_t)g & 1u, abort_flag)) break;
          tc05::tc_fence_after_sync();
          if (!issue_scores(n, g + 1)) break;
        }
        c = n;
      }
    }
  } else {
    // -------------------------------------------------------------------------- softmax warps
    // Per query tile: read S and dP, release them, form P and dS in registers while the tensor
    // cores still work on the previous tile's dV/dK/dQ; then hand P/dS over through shared memory and
    // add the previous dQ tile to global memory.  At the first tile of a new item the previous item's
    // dK and dV are taken out of tensor memory before P/dS are released (the new item's products
    // overwrite them) and stored while those products run.
    const int lg = warp & 3;          // tensor-memory lane group
    const int half = warp >> 2;       // which 64 key columns / which 32 dQ and dK/dV columns
    const int r = lg * 32 + lane;     // row within the tile
    const uint32_t lane_sel = (uint32_t)(lg * 32) << 16;
    bool ok = !*abort_flag;
    // dQ tile number `g` of the sequence, for query position t of (b, h): out of tensor memory and into the f32
    // accumulator in global memory
    // The tile is staged in shared memory and added by TMA reductions: 32 KB of f32 per query tile would otherwise
    // leave as 16-byte reductions issued by these warps, which then wait behind them.  Rows past T are clipped by the
    // tensor map.  Every warp stages its own 32 rows x 32 columns (4 KB, rows of 128 bytes, 128-byte swizzle) and its lane 0 adds
    // them with one TMA reduction of its own: no warp waits for another one, and the only wait is the lane's own, for
    // its previous reduction to have read the 4 KB, a whole tile earlier.
    uint8_t* my_stage = sdq + half * (FB_BM * 128) + lg * (32 * 128);
    auto add_dq_begin = [&](int g, uint32_t (&qb)[32]) {  // the tile starts to travel out of tensor memory
      tc05::tmem_ld_32x32b_x32(tmem_dq + (uint32_t)((g & 1) * 64) + lane_sel + half * 32, qb);
    };
    auto add_dq_finish = [&](const FbCursor& c, uint32_t (&qb)[32]) -> bool {
      if (lane == 0) tc05::tma_store_wait_read();  // this warp's previous reduction has read the staging rows
      tc05::tmem_ld_wait();
      tc05::tmem_ld_fence(qb);
      __syncwarp();
      uint8_t* line = my_stage + lane * 128;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        *reinterpret_cast<uint4*>(line + ((i ^ (lane & 7)) << 4)) = make_uint4(qb[i * 4], qb[i * 4 + 1], qb[i * 4 + 2], qb[i * 4 + 3]);
      tc05::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int t0 = (c.kj + c.it) * FB_BM + lg * 32;
        tc05::tma_reduce_add_3d(&map_dq, my_stage, c.h * FB_HD + c.cb * 64 + half * 32, t0, c.b);
        tc05::tma_store_commit();
      }
      return true;
    };
    // dV and dK of this thread's key row (32 columns each) out of tensor memory, already rounded to bf16 pairs:
    // words 0-15 hold dV, words 16-31 dK
    auto load_dkv = [&](uint32_t (&w)[32]) {
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        uint32_t raw[32];
        tc05::tmem_ld_32x32b_x32((which == 0 ? tmem_dv : tmem_dk) + lane_sel + half * 32, raw);
        tc05::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) w[which * 16 + i / 2] = pack_bf16x2(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
      }
    };
    // dK, dV of item c (row r = key): through the warp's staging rows (two tiles of 32 rows x 64 bytes, 64-byte
    // swizzle) and out with one TMA store each, 128-byte row segments together with the other half's warp, instead of
    // sixteen 16-byte stores a thread that each touch 32 different lines.  Keys past T are clipped by the tensor map.
    auto store_dkv = [&](const uint32_t (&w)[32], const FbCursor& c) {
      if (lane == 0) tc05::tma_store_wait_read();  // the dQ reduction queued just before has read the staging rows
      __syncwarp();
      uint8_t* tv = my_stage + lane * 64;
      uint8_t* tk = my_stage + 2048 + lane * 64;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int off = (i ^ ((lane >> 1) & 3)) << 4;
        *reinterpret_cast<uint4*>(tv + off) = make_uint4(w[i * 4], w[i * 4 + 1], w[i * 4 + 2], w[i * 4 + 3]);
        *reinterpret_cast<uint4*>(tk + off) = make_uint4(w[16 + i * 4], w[16 + i * 4 + 1], w[16 + i * 4 + 2], w[16 + i * 4 + 3]);
      }
      tc05::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int col = c.h * FB_HD + c.cb * 64 + half * 32, key0 = c.kj * FB_BN + lg * 32;
        tc05::tma_store_3d(&map_dv, my_stage, col, key0, c.b);
        tc05::tma_store_3d(&map_dk, my_stage + 2048, col, key0, c.b);
        tc05::tma_store_commit();
      }
    };
    // per-row statistics of a query tile, fetched one tile ahead
    // The two loads are requested here and their values first touched where the caller pins them (after the tile's
    // arithmetic), so that nothing waits for them on the way.
    auto row_stats = [&](const FbCursor& c, float* lse_raw, float* dlt_raw) {
      const int tt = c.valid() ? (c.kj + c.it) * FB_BM + r : 0;
      const bool in = c.valid() && tt < p.T;
      const size_t stat = in ? ((size_t)c.b * p.H + c.h) * p.T + tt : 0;
      *lse_raw = in ? __ldg(p.lse + stat) : INFINITY;  // rows past T: every P becomes 0
      *dlt_raw = in ? __ldg(p.delta + stat) : 0.f;
    };
    auto scale_stats = [&](float lse_raw, float dlt_raw, float* neg_lse2, float* neg_dlt_scaled) {
      *neg_lse2 = -lse_raw * 1.4426950408889634f;
      *neg_dlt_scaled = -dlt_raw * p.scale;
    };
    FbCursor c = first, prev = first;
    float neg_lse2, neg_dlt_scaled;
    {
      float l0, d0;
      row_stats(c, &l0, &d0);
      scale_stats(l0, d0, &neg_lse2, &neg_dlt_scaled);
    }
    int g = 0;
    // One query tile.  `Boundary` is the first tile of an item that follows another one: only that
    // instance carries the read-out of the previous item's dK and dV, so the steady-state instance
    // keeps its registers for the tile itself.
    auto tile = [&](auto boundary_tag, auto diag_tag) -> bool {
      constexpr bool Boundary = decltype(boundary_tag)::value;
      constexpr bool Diag = decltype(diag_tag)::value;
      const FbCursor n = fb_next(c, p);
      const int t = (c.kj + c.it) * FB_BM + r;  // query position
      const int key0 = c.kj * FB_BN;
      float next_lse_raw, next_dlt_raw;
      row_stats(n, &next_lse_raw, &next_dlt_raw);
      if (!tc05::mbar_wait(&bars->sdp_full, (uint32_t)g & 1u, abort_flag)) return false;
      tc05::tc_fence_after_sync();
      uint32_t pp[4][8], dd[4][8];  // P and dS of this thread's 64 key columns, bf16 pairs
      uint32_t sb[2][8], db[2][8];  // eight columns at a time, the next eight on their way
      tc05::tmem_ld_32x32b_x8(tmem_s + lane_sel + half * 64, sb[0]);
      tc05::tmem_ld_32x32b_x8(tmem_dp + lane_sel + half * 64, db[0]);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const int col0 = half * 64 + ch * 8;  // key column within the tile
        tc05::tmem_ld_wait();
        tc05::tmem_ld_fence(sb[ch & 1]);
        tc05::tmem_ld_fence(db[ch & 1]);
        if (ch < 7) {  // the next columns travel while these are worked on
          tc05::tmem_ld_32x32b_x8(tmem_s + lane_sel + col0 + 8, sb[(ch + 1) & 1]);
          tc05::tmem_ld_32x32b_x8(tmem_dp + lane_sel + col0 + 8, db[(ch + 1) & 1]);
        } else {  // all of S and dP is in registers: the next tile's may overwrite them
          tc05::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) tc05::mbar_arrive(&bars->sdp_free);
        }
        // P = 2^(S*scale*log2e - lse*log2e); rows past T carry lse = +inf, so their P is 0.  dS = P * (dP - D) * scale
        // with the scale folded into both terms.  Only the diagonal tile has keys above the query to mask.
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          float pr[2], dsv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float pv = ex2_fast(fmaf(__uint_as_float(sb[ch & 1][i + e]), p.scale_log2, neg_lse2));
            if constexpr (Diag) pv = (key0 + col0 + i + e > t) ? 0.f : pv;
            pr[e] = pv;
            dsv[e] = pv * fmaf(__uint_as_float(db[ch & 1][i + e]), p.scale, neg_dlt_scaled);
          }
          pp[ch / 2][(ch & 1) * 4 + i / 2] = pack_bf16x2(pr[0], pr[1]);
          dd[ch / 2][(ch & 1) * 4 + i / 2] = pack_bf16x2(dsv[0], dsv[1]);
        }
      }
      asm volatile("" : "+f"(next_lse_raw), "+f"(next_dlt_raw));  // first use of the loaded values: not before here
      scale_stats(next_lse_raw, next_dlt_raw, &neg_lse2, &neg_dlt_scaled);
      // the previous tile's products have finished: its dQ is ready and P/dS may be overwritten
      if (g > 0) {
        if (!tc05::mbar_wait(&bars->dq_full, (uint32_t)(g - 1) & 1u, abort_flag)) return false;
        tc05::tc_fence_after_sync();
      }
      uint8_t* pline = sp + half * (FB_BM * 128) + r * 128;
      uint8_t* dline = sds + half * (FB_BM * 128) + r * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int chunk = ch * 2 + q;  // 16-byte chunk = 8 keys
          const int off = (chunk ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(pline + off) = make_uint4(pp[ch][q * 4], pp[ch][q * 4 + 1], pp[ch][q * 4 + 2], pp[ch][q * 4 + 3]);
          *reinterpret_cast<uint4*>(dline + off) = make_uint4(dd[ch][q * 4], dd[ch][q * 4 + 1], dd[ch][q * 4 + 2], dd[ch][q * 4 + 3]);
        }
      }
      uint32_t dkv[Boundary ? 32 : 1];
      if constexpr (Boundary) load_dkv(dkv);  // before the new item's first products may overwrite them
      tc05::fence_proxy_async_smem();
      tc05::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&bars->p_full);
      // the other dQ buffer is not written again before this warp's next arrival on p_full
      // dK and dV first: the staging rows were last read a whole tile ago, so nothing waits; the dQ share that follows
      // waits only for these two plain stores to have read them
      if constexpr (Boundary) store_dkv(dkv, prev);
      if (g > 0) {
        uint32_t qb[32];
        add_dq_begin(g - 1, qb);
        if (!add_dq_finish(prev, qb)) return false;
      }
      prev = c;
      c = n;
      ++g;
      return true;
    };
    while (ok && c.valid()) {
      if (c.it == 0) ok = g > 0 ? tile(std::true_type{}, std::true_type{}) : tile(std::false_type{}, std::true_type{});
      else ok = tile(std::false_type{}, std::false_type{});
    }
    if (ok && g > 0) {  // dQ of the last query tile and dK, dV of the last item
      if (tc05::mbar_wait(&bars->dq_full, (uint32_t)(g - 1) & 1u, abort_flag)) {
        tc05::tc_fence_after_sync();
        uint32_t qb[32];
        add_dq_begin(g - 1, qb);
        add_dq_finish(prev, qb);
        uint32_t dkv[32];
        load_dkv(dkv);
        store_dkv(dkv, prev);
        if (lane == 0) tc05::tma_store_wait_all();  // the last reduction and stores have left shared memory and landed
      }
    }
  }

  tc05::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    if (threadIdx.x == 0) atomicExch(p.status + (layout_ok ? ST_WAIT_EXPIRED : ST_BAD_ARGUMENT), 1);
  }
  if (warp == FB_SOFTMAX_WARPS + 1) {
    tc05::tc_fence_after_sync();
    tc05::tmem_dealloc(tmem_s, FB_TMEM_COLS);
  }
}

// delta[b,h,t] = sum_j dO[b,t,h,j] * O[b,t,h,j]; eight lanes per (row, head), 16 bytes at a time.
__global__ void __launch_bounds__(256)
attention_delta_kernel(const __nv_bfloat16* __restrict__ out, long long ld_out, const __nv_bfloat16* __restrict__ dout,
                       long long ld_dout, float* __restrict__ delta, int B, int T, int H, int hd) {
  const long long pair = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 3;  // (row, head)
  const int part = threadIdx.x & 7;
  const bool in = pair < (long long)B * T * H;
  const int h = in ? (int)(pair % H) : 0;
  const long long row = in ? pair / H : 0;  // b*T + t
  float s = 0.f;
  for (int c = part * 8; c < hd; c += 64) {
    const uint4 o4 = *reinterpret_cast<const uint4*>(out + row * ld_out + h * hd + c);
    const uint4 d4 = *reinterpret_cast<const uint4*>(dout + row * ld_dout + h * hd + c);
    const float2 a0 = unpack_bf16x2(o4.x), a1 = unpack_bf16x2(o4.y), a2 = unpack_bf16x2(o4.z), a3 = unpack_bf16x2(o4.w);
    const float2 b0 = unpack_bf16x2(d4.x), b1 = unpack_bf16x2(d4.y), b2 = unpack_bf16x2(d4.z), b3 = unpack_bf16x2(d4.w);
    s += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (in && part == 0) {
    const int b = (int)(row / T), t = (int)(row % T);
    delta[((size_t)b * H + h) * T + t] = s;
  }
}

__global__ void dq_to_bf16_kernel(const float* __restrict__ acc, long long ld_acc, __nv_bfloat16* __restrict__ dq,
                                  long long ld_dq, long long rows, int cols) {
  const long long quads = rows * (cols / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < quads; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / (cols / 4);
    const int c = (int)(i % (cols / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(acc + row * ld_acc + c);
    *reinterpret_cast<uint2*>(dq + row * ld_dq + c) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
}

}  // namespace

size_t flash_attention_backward_scratch_bytes(int batch, int time, int n_heads, int head_dim) {
  const size_t rows = (size_t)batch * time;
  return sizeof(float) * rows * n_heads * head_dim + sizeof(float) * rows * n_heads + 256;
}

int flash_attention_backward_impl(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv,
                                  const void* out, long long ld_out, const void* dout, long long ld_dout,
                                  const float* lse, void* dq, void* dk, void* dv, long long ld_dqkv, int batch, int time,
                                  int n_heads, int head_dim, void* scratch, size_t scratch_bytes) {
  HL_REQUIRE(ctx && q && k && v && out && dout && lse && dq && dk && dv, "hl_flash_attention_backward: null argument");
  HL_REQUIRE(n_heads > 0 && batch > 0 && time > 0, "hl_flash_attention_backward: sizes must be positive");
  HL_REQUIRE(head_dim == 64 || head_dim == 128, "hl_flash_attention_backward: head_dim must be 64 or 128");
  const long long C = (long long)n_heads * head_dim;
  HL_REQUIRE(ld_qkv % 8 == 0 && ld_out % 8 == 0 && ld_dout % 8 == 0 && ld_dqkv % 8 == 0 && ld_qkv >= C && ld_out >= C &&
                 ld_dout >= C && ld_dqkv >= C,
             "hl_flash_attention_backward: row strides must be multiples of 8 and cover all heads");
  HL_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
               reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) |
               reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15) == 0,
             "hl_flash_attention_backward: pointers must be 16-byte aligned");
  const size_t rows = (size_t)batch * time;
  HL_REQUIRE(scratch && scratch_bytes >= flash_attention_backward_scratch_bytes(batch, time, n_heads, head_dim),
             "hl_flash_attention_backward: scratch is too small");
  float* dq_accum = reinterpret_cast<float*>(scratch);
  float* delta = dq_accum + rows * C;
  // five causal products against the forward's two
  ProfileScope prof(ctx, HL_PROF_ATTENTION_BWD, 5.0 * batch * n_heads * (double)time * time * head_dim);
  HL_CUDA(cudaMemsetAsync(dq_accum, 0, sizeof(float) * rows * C, ctx->stream));
  {
    const long long pairs = (long long)rows * n_heads;
    attention_delta_kernel<<<(unsigned)ceil_div_ll(pairs * 8, 256), 256, 0, ctx->stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), ld_out, reinterpret_cast<const __nv_bfloat16*>(dout), ld_dout,
        delta, batch, time, n_heads, head_dim);
    HL_LAUNCH_CHECK("attention_delta_kernel");
  }
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  // boxes of 64 channels (one 128-byte swizzle row); a head of 128 channels takes two boxes per tile
  if ((rc = make_tensor_map_bf16_2d(&mq, q, (uint64_t)C, rows, (uint64_t)ld_qkv, 64, FB_BM)) != HL_OK) return rc;
  if ((rc = make_tensor_map_bf16_2d(&mk, k, (uint64_t)C, rows, (uint64_t)ld_qkv, 64, FB_BN)) != HL_OK) return rc;
  if ((rc = make_tensor_map_bf16_2d(&mv, v, (uint64_t)C, rows, (uint64_t)ld_qkv, 64, FB_BN)) != HL_OK) return rc;
  if ((rc = make_tensor_map_bf16_2d(&mdo, dout, (uint64_t)C, rows, (uint64_t)ld_dout, 64, FB_BM)) != HL_OK) return rc;
  FbParams p{};
  p.B = batch; p.T = time; p.H = n_heads;
  p.blocks = head_dim / 64;
  p.lse = lse; p.delta = delta;
  p.dq_accum = dq_accum; p.ld_dq = C;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.ld_dkv = ld_dqkv;
  p.scale = 1.0f / sqrtf((float)head_dim);
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.status = ctx->status_dev;
  const int nq = ceil_div(time, FB_BM);
  // dQ accumulator as [batch][time][channels] f32, so that a tile's rows past `time` are clipped instead of landing in
  // the next batch entry; boxes of 32 columns (128 bytes) by 32 rows
  CUtensorMap mdq;
  {
    const uint64_t dims[3] = {(uint64_t)C, (uint64_t)time, (uint64_t)batch};
    const uint64_t strides[2] = {(uint64_t)C * sizeof(float), (uint64_t)time * (uint64_t)C * sizeof(float)};
    const uint32_t box[3] = {32, 32, 1};  // one softmax warp's share of a dQ tile
    if ((rc = make_tensor_map(&mdq, HL_F32, 3, dq_accum, dims, strides, box, 128)) != HL_OK) return rc;
  }
  // dK and dV as [batch][time][channels] bf16 with the caller's row stride; boxes of 32 channels (64 bytes) by 32 keys
  CUtensorMap mdk, mdv;
  {
    const uint64_t dims[3] = {(uint64_t)C, (uint64_t)time, (uint64_t)batch};
    const uint64_t strides[2] = {(uint64_t)ld_dqkv * 2, (uint64_t)time * (uint64_t)ld_dqkv * 2};
    const uint32_t box[3] = {32, 32, 1};
    if ((rc = make_tensor_map(&mdk, HL_BF16, 3, dk, dims, strides, box, 64)) != HL_OK) return rc;
    if ((rc = make_tensor_map(&mdv, HL_BF16, 3, dv, dims, strides, box, 64)) != HL_OK) return rc;
  }
  const int grid = std::min(nq * batch * n_heads * p.blocks, persistent_sms(ctx));
  if (head_dim == 64) {
    static bool configured = false;
    if (!configured) {
      HL_CUDA(cudaFuncSetAttribute(flash_attention_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FbSizes<64>::SMEM_BYTES));
      configured = true;
    }
    flash_attention_bwd_kernel<64><<<grid, FB_THREADS, FbSizes<64>::SMEM_BYTES, ctx->stream>>>(mq, mk, mv, mdo, mdq, mdk, mdv, p);
  } else {
    static bool configured = false;
    if (!configured) {
      HL_CUDA(cudaFuncSetAttribute(flash_attention_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FbSizes<128>::SMEM_BYTES));
      configured = true;
    }
    flash_attention_bwd_kernel<128><<<grid, FB_THREADS, FbSizes<128>::SMEM_BYTES, ctx->stream>>>(mq, mk, mv, mdo, mdq, mdk, mdv, p);
  }
  HL_LAUNCH_CHECK("flash_attention_bwd_kernel");
  {
    const long long quads = (long long)rows * (C / 4);
    const long long want = ceil_div_ll(quads, 256), cap = (long long)ctx->sm_count * 8;
    dq_to_bf16_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, ctx->stream>>>(
        dq_accum, C, reinterpret_cast<__nv_bfloat16*>(dq), ld_dqkv, (long long)rows, (int)C);
    HL_LAUNCH_CHECK("dq_to_bf16_kernel");
  }
  count_launch(ctx, 3);
  ctx->counters.attention_launches += 1;
  return HL_OK;
}

}  // namespace hl

extern "C" int hl_flash_attention_backward(hl_ctx* ctx, const void* q, const void* k, const void* v, long long ld_qkv,
                                           const void* out, long long ld_out, const void* dout, long long ld_dout,
                                           const float* lse, void* dq, void* dk, void* dv, long long ld_dqkv, int batch,
                                           int time, int n_heads, int head_dim) {
  if (!ctx) return hl::fail("hl_flash_attention_backward: null context");
  if (batch <= 0 || time <= 0 || n_heads <= 0 || head_dim <= 0)
    return hl::fail("hl_flash_attention_backward: sizes must be positive");
  const size_t need = hl::flash_attention_backward_scratch_bytes(batch, time, n_heads, head_dim);
  int rc = hl::ensure_workspace(ctx, need);
  if (rc != HL_OK) return rc;
  return hl::flash_attention_backward_impl(ctx, q, k, v, ld_qkv, out, ld_out, dout, ld_dout, lse, dq, dk, dv, ld_dqkv,
                                           batch, time, n_heads, head_dim, ctx->workspace, ctx->workspace_bytes);
}

