// bf16 x bf16 -> f32 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory, operands staged by TMA), one persistent warp-specialised kernel family.
//
// Replaces the reference's mma.sync tiers (heirloom-kernels/src/ptx/tensor_core.ptx:42-1527,
// wrappers heirloom-kernels/src/cuda.rs:4215-4386) together with the cast / transpose / pad /
// crop / bias kernels it launches around every matmul (src/nn.rs:432-446,
// src/tensor/autograd.rs:795-850): operand majors are expressed in the TMA descriptors, ragged
// edges by TMA zero fill on loads and clipping on stores, and bias / GELU / residual / dGELU run
// in the epilogue on the f32 accumulators.
//
// Tile: 128 (M) x 256 (N) x 64 (K) per stage, 4 stages (192 KB shared memory), two
// accumulator buffers of 256 tensor-memory columns so the epilogue of tile i overlaps the
// main loop of tile i+1.  Warp roles: warp 0 TMA producer, warp 1 MMA issuer (one elected
// thread), warps 2-9 epilogue: two warps per tensor-memory lane group, each taking 128 of the
// 256 columns.  An epilogue warp moves its 32 rows through two alternating 2 KB swizzled staging
// tiles and writes them with TMA stores (64-byte row segments, clipped at the tensor edge).
//
// Kernels: the generic one reads epilogue, output type and work split from its parameters; the training step's
// whole-tile products also have kernels compiled for their one epilogue and output type (template parameter SPEC), whose
// epilogue warps run straight-line code.
//
// Contractions of 2048 and up and the wide forward products, with whole tiles (or equal splits), run on pairs of CTAs: a
// cluster of two
// neighbouring SMs works on a 256 x 256 tile, the even CTA's MMA warp issues tcgen05.mma.cta_group::2 for both, each CTA
// stages its own 128 rows of A and 128 of B's 256 columns (six 32 KB stages in the same shared memory) and keeps its 128
// accumulator rows in its own tensor memory, so each SM reads half as much of B per MMA.  The even CTA's `full` barriers
// count both CTAs' TMA bytes, its `tmem_empty` barriers both CTAs' epilogue warps; MMA commits arrive in both CTAs.
//
// Tile order: round-robin over the CTAs; beside another stream's kernels (collectives in flight) the whole tiles of
// single CTAs are drawn from a counter instead, so a CTA that starts late takes fewer tiles (see `dyn` in the kernel).
//
// Work split: whole waves of output tiles go one tile per CTA; when the tiles left over would fill
// only part of a wave, their k blocks are dealt out evenly instead (every CTA gets one contiguous
// range of k blocks).  The CTA that owns the end of a tile's contraction
// finishes it: the others leave their raw accumulators in a per-CTA slot of a scratch area and
// raise a per-warp flag, and the finisher adds those slots in ascending CTA order before the
// normal epilogue, so the result does not depend on timing.  Slots are written before a CTA
// starts the range it finishes, so no CTA ever waits for one that is itself waiting.
#include <atomic>

#include "kernels.h"
#include "tc05.cuh"

namespace hl {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int MAX_STAGES = 6;
// CTA pairs: two CTAs of a cluster on one 256 x 256 tile, each staging its 128 rows of A and 128 of B's 256 columns, so
// a stage is 32 KB, six of them fit, and every SM reads half as much of B out of shared memory per MMA.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_STAGE_BYTES = B_STAGE_BYTES / 2;
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_B_STAGE_BYTES;
static_assert(PAIR_STAGES * PAIR_STAGE_BYTES <= STAGES * (A_STAGE_BYTES + B_STAGE_BYTES), "pair stages must fit the same shared memory");
constexpr int EPI_WARPS = 8;
constexpr int SCHED_SLOTS = 4;
constexpr int GEMM_THREADS = (2 + EPI_WARPS) * 32;
constexpr int TMEM_COLS = 512;
constexpr int STAGING_BYTES = 4096;  // per epilogue warp: two tiles of 32 rows x 64 bytes
constexpr size_t GEMM_SMEM_BYTES =
    size_t(STAGES) * STAGE_BYTES + size_t(EPI_WARPS) * STAGING_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

struct GemmParams {
  int m, n, k;
  int m_tiles, n_tiles, splits, k_blocks, k_blocks_per_split;
  int epilogue;
  int out_dtype;
  int partial_out;  // split-K: raw accumulators go to the [splits][m][n] scratch through map_c
  int dp_tiles, sk_tiles;   // whole-wave tiles, then tiles whose k blocks are dealt out evenly
  int panel_w;              // tile columns per panel of the tile order
  int a_kb_wrap;            // > 0: A holds this many k blocks and is read again from its start after them
  int b_kb_wrap;            // the same for B
  unsigned long long wait_limit_ns;  // bound of every pipeline wait
  int skip_kblock;          // test hook: the producer leaves out this k block of its first tile (-1: none)
  float* sk_slots;          // [grid][BM][BN] raw accumulators of unfinished tile parts
  unsigned* sk_flags;       // [grid][EPI_WARPS]: launch number once the warp's part of the slot is written
  unsigned sk_seq;          // this launch's number
  unsigned* sched;          // dynamic tile order: a counter that every processed tile advances by one; null: round-robin
  unsigned sched_base;      // the counter's value when this launch starts (the host adds each launch's tile count)
  long long ld_aux_in;
  const float* bias;
  const void* aux_in;
  int* status;
};

struct SharedTail {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sched_full[SCHED_SLOTS];   // dynamic tile order: the producer warp's thread hands the items to the other roles
  uint64_t sched_empty[SCHED_SLOTS];
  int sched_item[SCHED_SLOTS];
  uint32_t tmem_base;
  int abort_flag;
};

enum { ITEM_FULL = 0, ITEM_PART = 1, ITEM_FINISH = 2 };
struct WorkItem {
  int m_tile, n_tile, split, kb0, kb1;
  int kind;           // ITEM_FULL: whole contraction; ITEM_PART: leave raw sums in this CTA's slot;
                      // ITEM_FINISH: end of the contraction, add the slots of CTAs first_part .. blockIdx.x-1
  int first_part;
};

// Whether CTA `c` owns any k blocks of the evenly dealt region (with few units some CTAs own none).
__device__ __forceinline__ bool cta_has_units(const GemmParams& p, int c) {
  const long long units = (long long)p.sk_tiles * p.k_blocks;
  return c * units / (int)gridDim.x != (c + 1) * units / (int)gridDim.x;
}

// Which worker this CTA is and how many there are: a CTA, or a pair of CTAs that walks its tiles together.
template <bool PAIR>
__device__ __forceinline__ int worker_count() { return PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x; }
template <bool PAIR>
__device__ __forceinline__ int worker_index() { return PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x; }

// The `local`-th work item of this CTA, the same sequence for every warp role.
template <bool PAIR = false>
__device__ __forceinline__ bool get_item(const GemmParams& p, int local, WorkItem& w) {
  const int grid = worker_count<PAIR>(), cta = worker_index<PAIR>();
  const int tiles = p.m_tiles * p.n_tiles;
  w.split = 0;
  w.first_part = cta;
  int tile;
  if (p.sk_tiles == 0) {  // tiles (times explicit splits) round-robin, or handed out by a counter (item < 0: local is the item)
    const int item = local < 0 ? -local - 1 : cta + local * grid;
    if (item >= tiles * p.splits) return false;
    w.split = item / tiles;
    tile = item - w.split * tiles;
    w.kb0 = w.split * p.k_blocks_per_split;
    w.kb1 = min(p.k_blocks, w.kb0 + p.k_blocks_per_split);
    w.kind = ITEM_FULL;
  } else {
    const int n_dp = cta < p.dp_tiles ? (p.dp_tiles - cta + grid - 1) / grid : 0;
    if (local < n_dp) {
      tile = cta + local * grid;
      w.kb0 = 0;
      w.kb1 = p.k_blocks;
      w.kind = ITEM_FULL;
    } else {
      const int j = local - n_dp;
      const long long units = (long long)p.sk_tiles * p.k_blocks;
      const int u0 = (int)(cta * units / grid), u1 = (int)((cta + 1) * units / grid);
      if (u0 >= u1) return false;
      // The range covers the tail of one tile, whole tiles, and the head of one more.  Only the last
      // piece can stop short of its tile's end; it goes first, so that its slot is ready early, and
      // the piece that may have to wait for other CTAs' slots goes last.
      const int t_first = u0 / p.k_blocks, t_last = (u1 - 1) / p.k_blocks;
      const int n = t_last - t_first + 1;
      if (j >= n) return false;
      const bool last_is_part = (u1 % p.k_blocks) != 0;
      int t;
      if (last_is_part && n > 1) t = (j == 0) ? t_last : (j == n - 1 ? t_first : t_first + j);
      else t = (j == n - 1) ? t_first : t_first + 1 + j;
      const int lo = max(u0, t * p.k_blocks), hi = min(u1, (t + 1) * p.k_blocks);
      w.kb0 = lo - t * p.k_blocks;
      w.kb1 = hi - t * p.k_blocks;
      tile = p.dp_tiles + t;
      if (w.kb1 < p.k_blocks) {
        w.kind = ITEM_PART;
      } else if (w.kb0 == 0) {
        w.kind = ITEM_FULL;
      } else {
        w.kind = ITEM_FINISH;
        int first = cta;  // CTAs whose range reaches into this tile
        while (first > 0 && (long long)first * units / grid > (long long)t * p.k_blocks) --first;
        w.first_part = first;
      }
    }
  }
  // Tile order: panels of `panel_w` tile columns, rows of the panel one after the other.  CTAs that
  // run at the same time then share a few A row blocks and a few B column blocks, so each operand
  // byte comes out of DRAM once instead of once per tile column.
  const int per_panel = p.panel_w * p.m_tiles;
  const int panel = tile / per_panel;
  const int r = tile - panel * per_panel;
  const int width = min(p.panel_w, p.n_tiles - panel * p.panel_w);
  w.m_tile = r / width;
  w.n_tile = panel * p.panel_w + (r - w.m_tile * width);
  return true;
}

// SPEC < 0: epilogue, output type and work split are read from the parameters at run time.  SPEC >= 0: a product of whole
// tiles whose epilogue (SPEC / 2) and output type (SPEC & 1: bf16) are fixed at compile time, so that an epilogue warp
// runs straight-line code of its own variant only (the step's short-contraction products are bound by their epilogue);
// SPEC_PARTIAL: equal splits of the contraction whose raw f32 sums go to the scratch of the second kernel.
constexpr int SPEC_PARTIAL = 16;
template <bool A_MN, bool B_MN, bool PAIR, int SPEC>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_aux,
                         const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int NSTAGES = PAIR ? PAIR_STAGES : STAGES;
  constexpr int ST_BYTES = PAIR ? PAIR_STAGE_BYTES : STAGE_BYTES;  // one stage of this CTA
  constexpr int TILE_M = PAIR ? 2 * BM : BM;                       // rows of a work item
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;                       // columns of B this CTA stages
  uint8_t* staging_base = smem + size_t(STAGES) * STAGE_BYTES;     // same place whatever the stage count
  SharedTail* tail = reinterpret_cast<SharedTail*>(staging_base + size_t(EPI_WARPS) * STAGING_BYTES);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // In a pair the even CTA leads: its `full` barriers count the bytes of both CTAs' loads, its `tmem_empty` barriers
  // the epilogue warps of both; `empty` and `tmem_full` are signalled in each CTA by the leader's MMA commits.
  const uint32_t rank = PAIR ? tc05::cluster_cta_rank() : 0u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) {
      tc05::mbar_init(&tail->full[s], 1);
      tc05::mbar_init(&tail->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc05::mbar_init(&tail->tmem_full[b], 1);
      tc05::mbar_init(&tail->tmem_empty[b], PAIR ? 2 * EPI_WARPS : EPI_WARPS);
    }
    for (int q = 0; q < SCHED_SLOTS; ++q) {
      tc05::mbar_init(&tail->sched_full[q], 1);
      tc05::mbar_init(&tail->sched_empty[q], 1 + EPI_WARPS);  // the MMA issuer and every epilogue warp read an item
    }
    tail->abort_flag = 0;
    tc05::fence_barrier_init();
  }
  if (warp == 1) {
    if (PAIR) { tc05::tmem_alloc_pair(&tail->tmem_base, TMEM_COLS); tc05::tmem_relinquish_pair(); }
    else      { tc05::tmem_alloc(&tail->tmem_base, TMEM_COLS); tc05::tmem_relinquish(); }
  }
  tc05::tc_fence_before_sync();
  if (PAIR) tc05::cluster_sync_all(); else __syncthreads();
  tc05::tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;
  // Dynamic tile order: the first item of a CTA is its own index, every further one comes from a counter, so a CTA that
  // starts late (its SM was busy with another stream's kernel) simply takes fewer tiles and nobody waits for it.  The
  // producer warp's thread draws the items and hands them to the other roles through a small ring in shared memory.
  const bool dyn = !PAIR && p.sched != nullptr;
  const int items_total = p.m_tiles * p.n_tiles * p.splits;
  // (MMA issuer and epilogue warps) the `local`-th item of this CTA, -1 at the end, -2 when the wait ran out
  auto fetch_item = [&](int local, bool whole_warp) -> int {
    const int slot = local % SCHED_SLOTS;
    const uint32_t sphase = (uint32_t)(local / SCHED_SLOTS) & 1u;
    if (!tc05::mbar_wait(&tail->sched_full[slot], sphase, abort_flag, p.wait_limit_ns)) return -2;
    const int item = tail->sched_item[slot];
    if (whole_warp) __syncwarp();
    if (!whole_warp || lane == 0) tc05::mbar_arrive(&tail->sched_empty[slot]);
    return item;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (tc05::elect_one()) {
      tc05::tma_prefetch_desc(&map_a);
      tc05::tma_prefetch_desc(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkItem w;
      int item = worker_index<PAIR>();
      for (int local = 0; ok; ++local) {
        unsigned next_item = 0;
        if (dyn) {
          const int slot = local % SCHED_SLOTS;
          const uint32_t sphase = (uint32_t)(local / SCHED_SLOTS) & 1u;
          if (!tc05::mbar_wait(&tail->sched_empty[slot], sphase ^ 1u, abort_flag, p.wait_limit_ns)) { ok = false; break; }
          const bool more = item < items_total;
          tail->sched_item[slot] = more ? item : -1;
          tc05::mbar_arrive(&tail->sched_full[slot]);
          if (!more) break;
          get_item<false>(p, -item - 1, w);
          // asked for now, needed when this tile's loads are queued; unsigned arithmetic, the counter may wrap
          next_item = atomicAdd(p.sched, 1u) - p.sched_base + gridDim.x;
        } else if (!get_item<PAIR>(p, local, w)) {
          break;
        }
        const int m_row = w.m_tile * TILE_M + (int)rank * BM;      // this CTA's 128 rows of A
        const int n_row = w.n_tile * BN + (int)rank * B_ROWS;      // this CTA's columns of B
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!tc05::mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, p.wait_limit_ns)) { ok = false; break; }
          if (local == 0 && kb == p.skip_kblock) {  // test hook: this stage is never filled, the MMA issuer's wait runs out
            if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          uint8_t* sa = smem + size_t(stage) * ST_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          const int ka = p.a_kb_wrap > 0 ? kb % p.a_kb_wrap : kb;
          const int kbb = p.b_kb_wrap > 0 ? kb % p.b_kb_wrap : kb;
          if (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier; only the leader announces them
            const uint32_t bar = tc05::cluster_map_shared(&tail->full[stage], 0);
            if (rank == 0) tc05::mbar_arrive_expect_tx(&tail->full[stage], 2 * ST_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tc05::tma_load_2d_pair(sa + j * (BK * 128), &map_a, bar, m_row + j * 64, ka * BK);
            } else {
              tc05::tma_load_2d_pair(sa, &map_a, bar, ka * BK, m_row);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < B_ROWS / 64; ++j)
                tc05::tma_load_2d_pair(sb + j * (BK * 128), &map_b, bar, n_row + j * 64, kbb * BK);
            } else {
              tc05::tma_load_2d_pair(sb, &map_b, bar, kbb * BK, n_row);
            }
          } else {
            tc05::mbar_arrive_expect_tx(&tail->full[stage], ST_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tc05::tma_load_2d(sa + j * (BK * 128), &map_a, &tail->full[stage], m_row + j * 64, ka * BK);
            } else {
              tc05::tma_load_2d(sa, &map_a, &tail->full[stage], ka * BK, m_row);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tc05::tma_load_2d(sb + j * (BK * 128), &map_b, &tail->full[stage], n_row + j * 64, kbb * BK);
            } else {
              tc05::tma_load_2d(sb, &map_b, &tail->full[stage], kbb * BK, n_row);
            }
          }
          if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
        }
        item = (int)next_item;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (rank == 0 && tc05::elect_one()) {
      constexpr uint32_t idesc = tc05::instr_desc_bf16_f32(TILE_M, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkItem w;
      for (int local = 0; ok; ++local) {
        if (dyn) {
          const int item = fetch_item(local, false);
          if (item < 0) { ok = item == -1; break; }
          get_item<false>(p, -item - 1, w);
        } else if (!get_item<PAIR>(p, local, w)) {
          break;
        }
        const int kb0 = w.kb0, kb1 = w.kb1;
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        if (!tc05::mbar_wait(&tail->tmem_empty[buf], buf_phase ^ 1u, abort_flag, p.wait_limit_ns)) { ok = false; break; }
        tc05::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!tc05::mbar_wait(&tail->full[stage], phase, abort_flag, p.wait_limit_ns)) { ok = false; break; }
          tc05::tc_fence_after_sync();
          const uint32_t sa = tc05::smem_u32(smem + size_t(stage) * ST_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            const uint64_t da = A_MN ? tc05::smem_desc_sw128(sa + ks * (UMMA_K * 128), BK * 128, 1024)
                                     : tc05::smem_desc_sw128(sa + ks * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? tc05::smem_desc_sw128(sb + ks * (UMMA_K * 128), BK * 128, 1024)
                                     : tc05::smem_desc_sw128(sb + ks * (UMMA_K * 2), 16, 1024);
            if (PAIR) tc05::umma_ss_pair(tmem_d, da, db, idesc, (kb > kb0 || ks > 0) ? 1u : 0u);
            else      tc05::umma_ss(tmem_d, da, db, idesc, (kb > kb0 || ks > 0) ? 1u : 0u);
          }
          // frees the stage once these MMAs retire (in a pair: in both CTAs)
          if (PAIR) {
            tc05::umma_commit_pair(tc05::cluster_map_shared(&tail->empty[stage], 0));
            tc05::umma_commit_pair(tc05::cluster_map_shared(&tail->empty[stage], 1));
          } else {
            tc05::umma_commit(&tail->empty[stage]);
          }
          if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if (PAIR) {
            tc05::umma_commit_pair(tc05::cluster_map_shared(&tail->tmem_full[buf], 0));
            tc05::umma_commit_pair(tc05::cluster_map_shared(&tail->tmem_full[buf], 1));
          } else {
            tc05::umma_commit(&tail->tmem_full[buf]);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..9
    const int ew = warp - 2;
    const int lane_group = warp & 3;  // tensor-memory lanes this warp may read
    const int half = ew >> 2;         // which 128 of the tile's 256 columns
    // Two 2 KB staging tiles per warp ([32 rows x 64 bytes], 64-byte swizzle), used in turn, so
    // a TMA store is still reading one tile while the next columns are written into the other.
    uint8_t* staging = staging_base + size_t(ew) * STAGING_BYTES;
    int stage_sel = 0;
    const int epi = SPEC == SPEC_PARTIAL ? HL_EPI_NONE : SPEC >= 0 ? SPEC / 2 : p.epilogue;
    const bool partial = SPEC == SPEC_PARTIAL ? true : SPEC >= 0 ? false : p.partial_out != 0;
    const bool out_bf16 = SPEC == SPEC_PARTIAL ? false : SPEC >= 0 ? (SPEC & 1) != 0 : (!partial && p.out_dtype == HL_BF16);
    const bool need_aux = !partial && (epi == HL_EPI_BIAS_RESIDUAL || epi == HL_EPI_DGELU);
    const bool need_bias = !partial && p.bias != nullptr;
    bool ok = true;
    WorkItem w;
    // the accumulator buffer goes back to the MMA issuer, which in a pair sits in the even CTA
    auto release_buffer = [&](int buf) {
      if (PAIR) tc05::mbar_arrive_cluster(tc05::cluster_map_shared(&tail->tmem_empty[buf], 0));
      else tc05::mbar_arrive(&tail->tmem_empty[buf]);
    };
    // The `local`-th item of this CTA into `dst`: 1 = there is one, 0 = the sequence is over, -1 = a wait ran out.
    auto take_item = [&](int local, WorkItem& dst) -> int {
      if (dyn) {
        const int item = fetch_item(local, true);
        if (item < 0) return item == -1 ? 0 : -1;
        get_item<false>(p, -item - 1, dst);
        return 1;
      }
      return get_item<PAIR>(p, local, dst) ? 1 : 0;
    };
    // Global reads of the epilogue are issued ahead of their use so that their latency hides behind the previous
    // tile's last chunk, the wait for the accumulator and the previous chunk's arithmetic: the warp's 128 bias values
    // sit four per lane and are handed around by shuffles, and the residual / pre-activation rows are fetched one
    // 32-column chunk ahead.  The next tile's item, bias and first rows are asked for before the current tile's last
    // chunk is worked on.
    auto fetch_aux_of = [&](const WorkItem& x, int chunk, uint4 (&dst)[4]) {
      const int xrow = x.m_tile * TILE_M + (int)rank * BM + lane_group * 32 + lane;
      const int xcol0 = x.n_tile * BN + half * 128;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int col = xcol0 + chunk * 32 + q * 8;
        dst[q] = make_uint4(0, 0, 0, 0);
        if (need_aux && xrow < p.m && col < p.n)
          dst[q] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.aux_in) +
                                                        (size_t)xrow * p.ld_aux_in + col));
      }
    };
    auto fetch_bias_of = [&](const WorkItem& x) -> float4 {
      const int xcol0 = x.n_tile * BN + half * 128;
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (need_bias && xcol0 + lane * 4 < p.n) b = __ldg(reinterpret_cast<const float4*>(p.bias + xcol0 + lane * 4));
      return b;
    };
    WorkItem wn;
    uint4 aux_a[4], aux_b[4];
    float4 bias_reg = make_float4(0.f, 0.f, 0.f, 0.f), bias_next = bias_reg;
    int have = take_item(0, w);
    if (have == 1) {
      bias_reg = fetch_bias_of(w);
      fetch_aux_of(w, 0, aux_a);
    }
    for (int local = 0; ok && have == 1; ++local) {
      int have_next = -2;  // not asked for yet
      auto ask_next = [&]() {  // the next item, its bias and its first rows (into the buffer the chunk loop is done with)
        have_next = take_item(local + 1, wn);
        if (have_next == 1) {
          bias_next = fetch_bias_of(wn);
          fetch_aux_of(wn, 0, aux_b);
        }
      };
      const int split = w.split, n_tile = w.n_tile, m_tile = w.m_tile;
      const int buf = local & 1;
      const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
      const int row0 = m_tile * TILE_M + (int)rank * BM + lane_group * 32;
      const int row = row0 + lane;
      const bool row_ok = row < p.m;
      const int half_col0 = n_tile * BN + half * 128;
      auto fetch_aux = [&](int chunk, uint4 (&dst)[4]) { fetch_aux_of(w, chunk, dst); };
      if (!tc05::mbar_wait(&tail->tmem_full[buf], buf_phase, abort_flag, p.wait_limit_ns)) { ok = false; break; }
      tc05::tc_fence_after_sync();
      const uint32_t taddr_row = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(lane_group * 32) << 16);
      if (SPEC < 0 && w.kind == ITEM_PART) {
        // Raw sums of a part of the contraction: this warp's 32 rows x 128 columns go to the CTA's slot.
        // The slot is laid out [warp][chunk][q][lane] in 16-byte units, i.e. in the order the registers
        // come out of tensor memory, so that every store (and the finisher's load) covers 512
        // consecutive bytes.
        float4* slot = reinterpret_cast<float4*>(p.sk_slots + (size_t)blockIdx.x * (BM * BN)) + (size_t)ew * (4 * 8 * 32) + lane;
#pragma unroll 1
        for (int chunk = 0; chunk < 4; ++chunk) {
          if (half_col0 + chunk * 32 >= p.n) break;
          uint32_t acc_bits[32];
          tc05::tmem_ld_32x32b_x32(taddr_row + (uint32_t)(half * 128 + chunk * 32), acc_bits);
          tc05::tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            __stcg(slot + (chunk * 8 + q) * 32,
                   make_float4(__uint_as_float(acc_bits[q * 4]), __uint_as_float(acc_bits[q * 4 + 1]),
                               __uint_as_float(acc_bits[q * 4 + 2]), __uint_as_float(acc_bits[q * 4 + 3])));
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          unsigned* flag = p.sk_flags + (size_t)blockIdx.x * EPI_WARPS + ew;
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(p.sk_seq) : "memory");
        }
        tc05::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_buffer(buf);
        ask_next();
        if (have_next < 0) ok = false;
        have = have_next;
        w = wn;
        bias_reg = bias_next;
#pragma unroll
        for (int q = 0; q < 4; ++q) aux_a[q] = aux_b[q];
        continue;
      }
      if (SPEC < 0 && w.kind == ITEM_FINISH) {
        // The same warp of every earlier CTA on this tile wrote exactly the rows and columns this warp adds.
        if (lane == 0) {
          const unsigned long long t0 = tc05::global_timer_ns();
          for (int c = w.first_part; c < (int)blockIdx.x && ok; ++c) {
            if (!cta_has_units(p, c)) continue;
            const unsigned* flag = p.sk_flags + (size_t)c * EPI_WARPS + ew;
            for (uint32_t spins = 0;; ++spins) {
              unsigned seen;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
              if (seen == p.sk_seq) break;
              if ((spins & 63u) == 63u) {
                if (*abort_flag || tc05::global_timer_ns() - t0 > p.wait_limit_ns) { *abort_flag = 1; ok = false; break; }
                __nanosleep(64);
              }
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
      }
      // Sixteen 32-bit words of this lane's row (32 bf16 or 16 f32) go to the free staging tile
      // and out through one TMA store; at most one earlier store may still be reading.
      auto emit = [&](const CUtensorMap* map, const uint32_t* w, int col) {
        if (lane == 0) tc05::tma_store_wait_read1();
        __syncwarp();
        uint8_t* tile = staging + stage_sel * (STAGING_BYTES / 2);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(tile + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) =
              make_uint4(w[q * 4], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
        tc05::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (partial) tc05::tma_store_3d(map, tile, col, row0, split);
          else tc05::tma_store_2d(map, tile, col, row0);
          tc05::tma_store_commit();
        }
        stage_sel ^= 1;
      };
      auto process = [&](int chunk, const uint4 (&aux)[4]) {
        const int col0 = half_col0 + chunk * 32;
        uint32_t acc_bits[32];
        tc05::tmem_ld_32x32b_x32(taddr_row + (uint32_t)(half * 128 + chunk * 32), acc_bits);
        tc05::tmem_ld_wait();
        if (SPEC < 0 && w.kind == ITEM_FINISH) {
#pragma unroll 1
          for (int c = w.first_part; c < (int)blockIdx.x; ++c) {
            if (!cta_has_units(p, c)) continue;
            const float4* part = reinterpret_cast<const float4*>(p.sk_slots + (size_t)c * (BM * BN)) +
                                 (size_t)(ew * 4 + chunk) * (8 * 32) + lane;
            float4 t[8];  // all eight requests leave before the first sum needs its data
#pragma unroll
            for (int q = 0; q < 8; ++q) t[q] = __ldcg(part + q * 32);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              acc_bits[q * 4] = __float_as_uint(__uint_as_float(acc_bits[q * 4]) + t[q].x);
              acc_bits[q * 4 + 1] = __float_as_uint(__uint_as_float(acc_bits[q * 4 + 1]) + t[q].y);
              acc_bits[q * 4 + 2] = __float_as_uint(__uint_as_float(acc_bits[q * 4 + 2]) + t[q].z);
              acc_bits[q * 4 + 3] = __float_as_uint(__uint_as_float(acc_bits[q * 4 + 3]) + t[q].w);
            }
          }
        }
        uint32_t packed[16], gelu_packed[16], hi_words[16];  // f32 output: packed = columns 0-15, hi_words = 16-31
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // groups of 8 columns
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc_bits[g * 8 + i]);
          if (!partial) {
            if (need_bias) {
              // columns chunk*32 + g*8 + i of this half live in lane chunk*8 + g*2 + i/4
              const int src = chunk * 8 + g * 2;
              v[0] += __shfl_sync(0xffffffffu, bias_reg.x, src); v[1] += __shfl_sync(0xffffffffu, bias_reg.y, src);
              v[2] += __shfl_sync(0xffffffffu, bias_reg.z, src); v[3] += __shfl_sync(0xffffffffu, bias_reg.w, src);
              v[4] += __shfl_sync(0xffffffffu, bias_reg.x, src + 1); v[5] += __shfl_sync(0xffffffffu, bias_reg.y, src + 1);
              v[6] += __shfl_sync(0xffffffffu, bias_reg.z, src + 1); v[7] += __shfl_sync(0xffffffffu, bias_reg.w, src + 1);
            }
            if (epi == HL_EPI_BIAS_GELU) {
              // h = bf16(acc + bias) is the main output; g = bf16(gelu(h)) the second one
              // rounded two at a time by the packing conversion (the packed word is the output word as well) and widened
              // again with one integer op each: a quarter of the instructions of rounding on integer ops
              float gl[8];
#pragma unroll
              for (int i = 0; i < 8; i += 2) {
                const uint32_t hw = pack_bf16x2(v[i], v[i + 1]);
                packed[g * 4 + i / 2] = hw;
                v[i] = __uint_as_float(hw << 16);
                v[i + 1] = __uint_as_float(hw & 0xFFFF0000u);
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) gl[i] = gelu_fwd_fast(v[i]);
              gelu_packed[g * 4] = pack_bf16x2(gl[0], gl[1]); gelu_packed[g * 4 + 1] = pack_bf16x2(gl[2], gl[3]);
              gelu_packed[g * 4 + 2] = pack_bf16x2(gl[4], gl[5]); gelu_packed[g * 4 + 3] = pack_bf16x2(gl[6], gl[7]);
            } else if (epi == HL_EPI_BIAS_RESIDUAL || epi == HL_EPI_DGELU) {
              const uint4 r = aux[g];
              const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
              const float rr[8] = {r0.x, r0.y, r1.x, r1.y, r2.x, r2.y, r3.x, r3.y};
              if (epi == HL_EPI_BIAS_RESIDUAL) {
                // out = bf16(residual + bf16(acc + bias)): the two round trips of the block
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                  const uint32_t hw = pack_bf16x2(v[i], v[i + 1]);
                  v[i] = rr[i] + __uint_as_float(hw << 16);
                  v[i + 1] = rr[i + 1] + __uint_as_float(hw & 0xFFFF0000u);
                }
              } else {
                // out = acc * gelu'(h), h read from aux_in
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = v[i] * gelu_grad_fast(rr[i]);
              }
            }
          }
          if (out_bf16 && epi == HL_EPI_BIAS_GELU) {  // h was packed when it was rounded
          } else if (out_bf16) {
            packed[g * 4] = pack_bf16x2(v[0], v[1]); packed[g * 4 + 1] = pack_bf16x2(v[2], v[3]);
            packed[g * 4 + 2] = pack_bf16x2(v[4], v[5]); packed[g * 4 + 3] = pack_bf16x2(v[6], v[7]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (g < 2) packed[g * 8 + i] = __float_as_uint(v[i]);
              else hi_words[(g - 2) * 8 + i] = __float_as_uint(v[i]);
            }
          }
        }
        if (out_bf16) {
          emit(&map_c, packed, col0);
          if (epi == HL_EPI_BIAS_GELU) emit(&map_aux, gelu_packed, col0);
        } else {
          emit(&map_c, packed, col0);
          if (col0 + 16 < p.n) emit(&map_c, hi_words, col0 + 16);
        }
      };
      // chunks beyond the matrix edge are skipped (the test is uniform across the warp)
#pragma unroll 1
      for (int chunk = 0; chunk < 4; ++chunk) {
        if (half_col0 + chunk * 32 >= p.n) break;
        const bool last = chunk == 3 || half_col0 + (chunk + 1) * 32 >= p.n;
        if (!last) fetch_aux(chunk + 1, aux_b);
        else ask_next();
        process(chunk, aux_a);
#pragma unroll
        for (int q = 0; q < 4; ++q) aux_a[q] = aux_b[q];
      }
      tc05::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) release_buffer(buf);
      if (have_next == -2) {  // no chunk of this half lies inside the matrix
        ask_next();
#pragma unroll
        for (int q = 0; q < 4; ++q) aux_a[q] = aux_b[q];
      }
      if (have_next < 0) ok = false;
      have = have_next;
      w = wn;
      bias_reg = bias_next;
    }
    if (lane == 0) tc05::tma_store_wait_all();  // global writes are complete before the kernel ends
  }

  // ---------------------------------------------------------------------- teardown
  tc05::tc_fence_before_sync();
  // In a pair neither CTA may leave (or free tensor memory) while the other still reads its shared memory through the
  // MMAs or arrives on its barriers; every loop above is bounded, so both get here.
  if (PAIR) tc05::cluster_sync_all(); else __syncthreads();
  if (*abort_flag) {
    // Give copies already in flight time to land before shared memory is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    if (threadIdx.x == 0) atomicExch(p.status + ST_WAIT_EXPIRED, 1);
  }
  if (warp == 1) {
    tc05::tc_fence_after_sync();
    if (PAIR) tc05::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tc05::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

__global__ void splitk_reduce_kernel(const float* __restrict__ partials, float* __restrict__ out, int m, int n,
                                     long long ldc, int splits) {
  const long long quads = (long long)m * (n / 4);
  for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < quads; q += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(q / (n / 4));
    const int c4 = (int)(q - (long long)row * (n / 4));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(partials + ((size_t)s * m + row) * (size_t)n) + c4);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)row * ldc + c4 * 4) = acc;
  }
}

template <bool A_MN, bool B_MN, bool PAIR, int SPEC = -1>
int launch_variant(hl_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                   const CUtensorMap& maux, const GemmParams& p, int grid) {
  auto kern = gemm_bf16_tcgen05_kernel<A_MN, B_MN, PAIR, SPEC>;
  static bool configured = false;
  if (!configured) {
    HL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_BYTES));
    configured = true;
  }
  if (PAIR) {
    // `grid` CTAs in clusters of two neighbouring SMs
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    // no more pairs than can be resident at once (a GPC with an odd number of free SMs leaves one out)
    static int resident_pairs = 0;
    if (resident_pairs == 0) {
      int n = 0;
      HL_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
      HL_REQUIRE(n > 0, "hl_gemm_bf16: no CTA pair fits on this device");
      resident_pairs = n;
    }
    if (grid > 2 * resident_pairs) cfg.gridDim = dim3((unsigned)(2 * resident_pairs));
    HL_CUDA(cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, maux, p));
  } else {
    kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, ctx->stream>>>(ma, mb, mc, maux, p);
  }
  HL_LAUNCH_CHECK("gemm_bf16_tcgen05_kernel");
  count_launch(ctx);
  ctx->counters.gemm_tcgen05_launches += 1;
  if (PAIR) ctx->counters.gemm_pair_launches += 1;
  return HL_OK;
}

// Which products run on CTA pairs: HEIRLOOM_GEMM_PAIRS=1 every whole-tile product, 0 none; unset, those with a contraction
// of kPairMinK and up and the wide forward products.  Read at every call.
constexpr int kPairMinK = 2048;
bool pairs_enabled(const hl_gemm_desc* d) {
  const char* e = getenv("HEIRLOOM_GEMM_PAIRS");
  if (e && e[0] == '1') return true;
  if (e && e[0] == '0') return false;
  if (d->k >= kPairMinK) return true;
  // Short contractions are bound by what the SMs can pull out of L2 (every tile reads its operands again: the MMA issuer
  // of the qkv forward product spends three quarters of a tile waiting for operand stages, not for the epilogue), and a
  // pair reads a third less per output.  It pays where the output is wide: qkv forward 51.3 -> 47.8 us, fc1 forward
  // 84.5 -> 81.5, lm_head forward 1290 -> 1230; the 768-wide outputs and the input gradients lose a few per cent.
  return d->a_layout == HL_K_MAJOR && d->b_layout == HL_K_MAJOR && d->n >= 2048 &&
         (d->epilogue == HL_EPI_BIAS || d->epilogue == HL_EPI_BIAS_GELU);
}

}  // namespace

constexpr int kMinDealtKBlocks = 192;  // contraction of 12288 and up

GemmPlan gemm_plan(const hl_gemm_desc* d, int sm_count) {
  GemmPlan plan{};
  const int m_tiles = ceil_div(d->m, BM), n_tiles = ceil_div(d->n, BN);
  const int k_blocks = ceil_div(d->k, BK);
  const int tiles = m_tiles * n_tiles;
  plan.splits = 1;
  plan.dp_tiles = tiles;
  if (d->split_k > 1) {
    // explicit request: every tile's contraction cut into equal parts, summed by a second kernel
    int splits = std::min(d->split_k, k_blocks);
    const int per = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, per);  // every split owns at least one k block
    plan.splits = splits;
    if (splits > 1) plan.splitk_bytes = (size_t)splits * d->m * (size_t)d->n * sizeof(float);
  } else if (d->split_k <= 0) {
    const int rem = tiles % sm_count, waves = tiles / sm_count;
    const bool plain_f32 = d->epilogue == HL_EPI_NONE && d->out_dtype == HL_F32;
    if (rem != 0 && rem * 100 < sm_count * 85 && waves < 8 && k_blocks >= kMinDealtKBlocks && tiles * 2 >= sm_count) {
      // A partly filled last wave of long tiles: deal out its k blocks.  When it is less than half
      // full, one whole wave joins it, so that a tile is never shared by more than three CTAs.  The
      // hand-over costs about 15 us per launch, so short contractions keep whole tiles.
      int sk = rem;
      if (rem * 2 < sm_count && waves >= 1) sk += sm_count;
      plan.dp_tiles = tiles - sk;
      plan.sk_tiles = sk;
      plan.sk_slot_bytes = (size_t)sm_count * BM * BN * sizeof(float);
    } else if (plain_f32 && tiles * 2 < sm_count && k_blocks >= 16) {
      // Few output tiles and a long contraction (weight gradients): equal splits with a second
      // kernel for the sums; pick the split that fills whole waves best.
      int splits = 1;
      double best = (double)tiles / (double)(ceil_div(tiles, sm_count) * sm_count);
      for (int s = 2; s <= 16 && k_blocks / s >= 8; ++s) {
        const int items = tiles * s;
        const double eff = (double)items / (double)(ceil_div(items, sm_count) * sm_count);
        if (eff > best + 0.02) { best = eff; splits = s; }
      }
      const int per = ceil_div(k_blocks, splits);
      splits = ceil_div(k_blocks, per);
      plan.splits = splits;
      if (splits > 1) plan.splitk_bytes = (size_t)splits * d->m * (size_t)d->n * sizeof(float);
    }
  }
  return plan;
}

size_t gemm_stream_flag_bytes(int sm_count) { return (size_t)sm_count * EPI_WARPS * sizeof(unsigned); }

static std::atomic<unsigned> g_stream_launch_number{0};

int gemm_bf16_run(hl_ctx* ctx, const hl_gemm_desc* d, const void* a, const void* b, void* c, const float* bias,
                  const void* aux_in, void* aux_out, float* workspace, size_t workspace_bytes, unsigned* stream_flags) {
  HL_REQUIRE(ctx && d, "hl_gemm_bf16: null argument");
  HL_REQUIRE(d->m > 0 && d->n > 0 && d->k > 0, "hl_gemm_bf16: m, n, k must be positive");
  HL_REQUIRE(a && b && c, "hl_gemm_bf16: null operand pointer");
  HL_REQUIRE(d->n % 8 == 0 && d->ldc % 8 == 0, "hl_gemm_bf16: n and ldc must be multiples of 8");
  HL_REQUIRE(d->lda % 8 == 0 && d->ldb % 8 == 0, "hl_gemm_bf16: lda and ldb must be multiples of 8 elements");
  HL_REQUIRE(d->out_dtype == HL_BF16 || d->out_dtype == HL_F32, "hl_gemm_bf16: output dtype must be bf16 or f32");
  HL_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(c) & 15) == 0,
             "hl_gemm_bf16: operands must be 16-byte aligned");
  const bool a_mn = d->a_layout == HL_MN_MAJOR, b_mn = d->b_layout == HL_MN_MAJOR;
  HL_REQUIRE(d->a_k_period >= 0 && d->a_k_period % BK == 0 && d->a_k_period <= d->k,
             "hl_gemm_bf16: a_k_period must be a multiple of 64 and at most k");
  HL_REQUIRE(d->b_k_period >= 0 && d->b_k_period % BK == 0 && d->b_k_period <= d->k,
             "hl_gemm_bf16: b_k_period must be a multiple of 64 and at most k");
  const int a_k = d->a_k_period > 0 ? d->a_k_period : d->k;  // contraction extent that A really holds
  const int b_k = d->b_k_period > 0 ? d->b_k_period : d->k;
  HL_REQUIRE(d->lda >= (a_mn ? d->m : a_k) && d->ldb >= (b_mn ? d->n : b_k) && d->ldc >= d->n,
             "hl_gemm_bf16: leading dimension smaller than the row length");
  const long long ld_aux_in = d->ld_aux_in > 0 ? d->ld_aux_in : d->ldc;
  const long long ld_aux_out = d->ld_aux_out > 0 ? d->ld_aux_out : d->ldc;
  switch (d->epilogue) {
    case HL_EPI_NONE: break;
    case HL_EPI_BIAS: HL_REQUIRE(bias, "hl_gemm_bf16: bias epilogue needs a bias"); break;
    case HL_EPI_BIAS_GELU:
      HL_REQUIRE(bias && aux_out && d->out_dtype == HL_BF16, "hl_gemm_bf16: bias+gelu needs bias, aux_out and bf16 output");
      HL_REQUIRE(ld_aux_out % 8 == 0 && ld_aux_out >= d->n && (reinterpret_cast<uintptr_t>(aux_out) & 15) == 0,
                 "hl_gemm_bf16: aux_out must be 16-byte aligned with a row stride that is a multiple of 8");
      break;
    case HL_EPI_BIAS_RESIDUAL:
      HL_REQUIRE(bias && aux_in && d->out_dtype == HL_BF16, "hl_gemm_bf16: bias+residual needs bias, aux_in and bf16 output");
      break;
    case HL_EPI_DGELU: HL_REQUIRE(aux_in, "hl_gemm_bf16: dgelu epilogue needs aux_in"); break;
    default: return fail("hl_gemm_bf16: unknown epilogue");
  }
  if (aux_in)
    HL_REQUIRE(ld_aux_in % 8 == 0 && ld_aux_in >= d->n && (reinterpret_cast<uintptr_t>(aux_in) & 15) == 0,
               "hl_gemm_bf16: aux_in must be 16-byte aligned with a row stride that is a multiple of 8");
  if (bias) HL_REQUIRE((reinterpret_cast<uintptr_t>(bias) & 15) == 0, "hl_gemm_bf16: bias must be 16-byte aligned");

  const int sms = persistent_sms(ctx);
  const GemmPlan plan = gemm_plan(d, sms);
  // Whole tiles (of the whole contraction or of equal splits of it; not the dealt-out k blocks) can run on CTA pairs
  // with 256-row tiles.  Measured on alternating calls: 6-7 % faster where the main loop bounds the tile (contractions
  // of 2304 and up), 6-10 % slower at 768, where the epilogue does and the leader waits for both CTAs' epilogue warps.
  const bool pair = pairs_enabled(d) && plan.sk_tiles == 0 && d->m > BM && sms >= 2 && ctx->gemm_skip_kblock < 0;
  GemmParams p{};
  p.m = d->m; p.n = d->n; p.k = d->k;
  p.m_tiles = ceil_div(d->m, pair ? 2 * BM : BM);
  p.n_tiles = ceil_div(d->n, BN);
  p.k_blocks = ceil_div(d->k, BK);
  // An A operand that stays in L2 anyway keeps the plain order (one tile column after the other);
  // a larger one is walked in panels of up to eight tile columns so that it streams from DRAM once.
  p.a_kb_wrap = d->a_k_period > 0 ? d->a_k_period / BK : 0;
  p.b_kb_wrap = d->b_k_period > 0 ? d->b_k_period / BK : 0;
  p.wait_limit_ns = ctx->wait_limit_ns ? ctx->wait_limit_ns : tc05::kWaitLimitNs;
  p.skip_kblock = ctx->gemm_skip_kblock;
  p.panel_w = (size_t)d->m * (size_t)d->k * 2 <= (size_t(32) << 20) ? 1 : std::min(p.n_tiles, 8);
  const int splits = plan.splits;
  const size_t need = plan.splitk_bytes;
  p.splits = splits;
  p.dp_tiles = plan.dp_tiles;
  p.sk_tiles = plan.sk_tiles;
  if (plan.sk_tiles > 0) {
    HL_REQUIRE(workspace != nullptr && workspace_bytes >= plan.sk_slot_bytes && stream_flags != nullptr,
               "hl_gemm_bf16: scratch for partly finished tiles is too small");
    HL_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "hl_gemm_bf16: scratch must be 16-byte aligned");
    p.sk_slots = workspace;
    p.sk_flags = stream_flags;
    unsigned seq = ++g_stream_launch_number;
    if (seq == 0) seq = ++g_stream_launch_number;  // 0 means "never written"
    p.sk_seq = seq;
  }
  // Beside another stream's kernels (collectives in flight) whole tiles and equal splits are handed out by a counter
  // instead of round-robin: per launch it costs about a microsecond, and it keeps a CTA that starts late from holding
  // up its share of the tiles.  HEIRLOOM_GEMM_DYNAMIC=1 / 0 forces it on / off.  Every tile advances the counter by
  // one, so the host knows its value at the start of the next launch without touching the device.
  {
    const char* e = getenv("HEIRLOOM_GEMM_DYNAMIC");
    const bool dynamic = e && (e[0] == '0' || e[0] == '1') ? e[0] == '1' : nccl_active(ctx);
    p.sched = (dynamic && !pair && plan.sk_tiles == 0 && ctx->gemm_skip_kblock < 0) ? ctx->gemm_sched : nullptr;
    if (p.sched) {
      p.sched_base = ctx->gemm_sched_base;  // advanced below, once the launch has been queued
    }
  }
  p.k_blocks_per_split = ceil_div(p.k_blocks, splits);
  p.epilogue = d->epilogue;
  p.out_dtype = d->out_dtype;
  p.ld_aux_in = ld_aux_in;
  p.bias = bias; p.aux_in = aux_in;
  p.status = ctx->status_dev;
  p.partial_out = 0;
  if (splits > 1) {
    HL_REQUIRE(d->epilogue == HL_EPI_NONE && d->out_dtype == HL_F32, "hl_gemm_bf16: split-K needs a plain f32 output");
    HL_REQUIRE(workspace != nullptr && workspace_bytes >= need, "hl_gemm_bf16: split-K scratch is too small");
    HL_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "hl_gemm_bf16: split-K scratch must be 16-byte aligned");
    p.partial_out = 1;
  }

  CUtensorMap ma, mb, mc, maux;
  int rc;
  if (a_mn) rc = make_tensor_map_bf16_2d(&ma, a, (uint64_t)d->m, (uint64_t)a_k, (uint64_t)d->lda, 64, BK);
  else      rc = make_tensor_map_bf16_2d(&ma, a, (uint64_t)a_k, (uint64_t)d->m, (uint64_t)d->lda, BK, BM);
  if (rc != HL_OK) return rc;
  if (b_mn) rc = make_tensor_map_bf16_2d(&mb, b, (uint64_t)d->n, (uint64_t)b_k, (uint64_t)d->ldb, 64, BK);
  else      rc = make_tensor_map_bf16_2d(&mb, b, (uint64_t)b_k, (uint64_t)d->n, (uint64_t)d->ldb, BK, pair ? BN / 2 : BN);
  if (rc != HL_OK) return rc;
  if (p.partial_out) {
    const uint64_t dims[3] = {(uint64_t)d->n, (uint64_t)d->m, (uint64_t)splits};
    const uint64_t strides[2] = {(uint64_t)d->n * 4, (uint64_t)d->n * (uint64_t)d->m * 4};
    const uint32_t box[3] = {16, 32, 1};
    rc = make_tensor_map(&mc, HL_F32, 3, workspace, dims, strides, box, 64);
  } else {
    const uint64_t dims[2] = {(uint64_t)d->n, (uint64_t)d->m};
    const uint64_t strides[1] = {(uint64_t)d->ldc * (d->out_dtype == HL_BF16 ? 2u : 4u)};
    const uint32_t box[2] = {d->out_dtype == HL_BF16 ? 32u : 16u, 32u};  // 64-byte rows
    rc = make_tensor_map(&mc, d->out_dtype, 2, c, dims, strides, box, 64);
  }
  if (rc != HL_OK) return rc;
  if (d->epilogue == HL_EPI_BIAS_GELU) {
    const uint64_t dims[2] = {(uint64_t)d->n, (uint64_t)d->m};
    const uint64_t strides[1] = {(uint64_t)ld_aux_out * 2};
    const uint32_t box[2] = {32, 32};
    rc = make_tensor_map(&maux, HL_BF16, 2, aux_out, dims, strides, box, 64);
    if (rc != HL_OK) return rc;
  } else {
    maux = mc;
  }

  const int total = p.m_tiles * p.n_tiles * p.splits;
  const int grid = pair ? 2 * min(total, sms / 2) : plan.sk_tiles > 0 ? sms : min(total, sms);
  ProfileScope prof(ctx, HL_PROF_GEMM, 2.0 * (double)d->m * (double)d->n * (double)d->k);
  // The training step's products with whole tiles have kernels of their own, compiled for one epilogue and output type.
  const bool simple = splits == 1 && plan.sk_tiles == 0;
  const int spec = simple ? d->epilogue * 2 + (d->out_dtype == HL_BF16 ? 1 : 0)
                          : (splits > 1 && plan.sk_tiles == 0) ? SPEC_PARTIAL : -1;
  constexpr int kBias = HL_EPI_BIAS * 2, kGelu = HL_EPI_BIAS_GELU * 2, kResidual = HL_EPI_BIAS_RESIDUAL * 2,
                kDgelu = HL_EPI_DGELU * 2, kNone = HL_EPI_NONE * 2;
  bool launched = true;
  if (!a_mn && !b_mn && !pair && spec == kBias + 1) rc = launch_variant<false, false, false, kBias + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && !b_mn && !pair && spec == kBias) rc = launch_variant<false, false, false, kBias>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && !b_mn && !pair && spec == kGelu + 1) rc = launch_variant<false, false, false, kGelu + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && !b_mn && !pair && spec == kResidual + 1) rc = launch_variant<false, false, false, kResidual + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && !b_mn && pair && spec == kResidual + 1) rc = launch_variant<false, false, true, kResidual + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && !b_mn && pair && spec == kBias + 1) rc = launch_variant<false, false, true, kBias + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && !b_mn && pair && spec == kGelu + 1) rc = launch_variant<false, false, true, kGelu + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && !b_mn && pair && spec == kBias) rc = launch_variant<false, false, true, kBias>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && b_mn && pair && spec == kDgelu + 1) rc = launch_variant<false, true, true, kDgelu + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && b_mn && pair && spec == kNone + 1) rc = launch_variant<false, true, true, kNone + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && b_mn && !pair && spec == kDgelu + 1) rc = launch_variant<false, true, false, kDgelu + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && b_mn && !pair && spec == kNone + 1) rc = launch_variant<false, true, false, kNone + 1>(ctx, ma, mb, mc, maux, p, grid);
  else if (!a_mn && b_mn && pair && spec == kNone) rc = launch_variant<false, true, true, kNone>(ctx, ma, mb, mc, maux, p, grid);
  else if (a_mn && b_mn && pair && spec == kNone) rc = launch_variant<true, true, true, kNone>(ctx, ma, mb, mc, maux, p, grid);
  else if (a_mn && b_mn && pair && spec == SPEC_PARTIAL) rc = launch_variant<true, true, true, SPEC_PARTIAL>(ctx, ma, mb, mc, maux, p, grid);
  else launched = false;
  if (launched) {
  } else if (pair) {
    if (a_mn && b_mn) rc = launch_variant<true, true, true>(ctx, ma, mb, mc, maux, p, grid);
    else if (a_mn)    rc = launch_variant<true, false, true>(ctx, ma, mb, mc, maux, p, grid);
    else if (b_mn)    rc = launch_variant<false, true, true>(ctx, ma, mb, mc, maux, p, grid);
    else              rc = launch_variant<false, false, true>(ctx, ma, mb, mc, maux, p, grid);
  } else {
    if (a_mn && b_mn) rc = launch_variant<true, true, false>(ctx, ma, mb, mc, maux, p, grid);
    else if (a_mn)    rc = launch_variant<true, false, false>(ctx, ma, mb, mc, maux, p, grid);
    else if (b_mn)    rc = launch_variant<false, true, false>(ctx, ma, mb, mc, maux, p, grid);
    else              rc = launch_variant<false, false, false>(ctx, ma, mb, mc, maux, p, grid);
  }
  if (rc != HL_OK) return rc;
  if (p.sched) ctx->gemm_sched_base += (unsigned)total;  // every tile of the launch draws from the counter once
  if (splits > 1) {
    const long long quads = (long long)d->m * (d->n / 4);
    const long long want_blocks = ceil_div_ll(quads, 256), cap_blocks = (long long)ctx->sm_count * 8;
    const int blocks = (int)(want_blocks < cap_blocks ? want_blocks : cap_blocks);
    splitk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(workspace, reinterpret_cast<float*>(c), d->m, d->n, d->ldc, splits);
    HL_LAUNCH_CHECK("splitk_reduce_kernel");
    count_launch(ctx);
  }
  return HL_OK;
}

}  // namespace hl

namespace hl {
int gemm_bf16_ctx(hl_ctx* ctx, const hl_gemm_desc* desc, const void* a, const void* b, void* c, const float* bias,
                  const void* aux_in, void* aux_out) {
  if (!ctx || !desc) return fail("hl_gemm_bf16: null argument");
  if (desc->m <= 0 || desc->n <= 0 || desc->k <= 0) return fail("hl_gemm_bf16: m, n, k must be positive");
  const GemmPlan plan = gemm_plan(desc, persistent_sms(ctx));
  const size_t need = std::max(plan.splitk_bytes, plan.sk_slot_bytes);
  if (need > ctx->workspace_bytes) {
    int rc = ensure_workspace(ctx, need);
    if (rc != HL_OK) return rc;
  }
  if (plan.sk_tiles > 0 && ctx->gemm_flags == nullptr) {
    // once per context: the flags have to start at zero and must survive growth of the scratch arena
    const size_t bytes = gemm_stream_flag_bytes(ctx->sm_count);
    HL_CUDA(cudaMalloc(&ctx->gemm_flags, bytes));
    HL_CUDA(cudaMemsetAsync(ctx->gemm_flags, 0, bytes, ctx->stream));
    ctx->counters.allocations += 1;
    ctx->counters.allocated_bytes += bytes;
  }
  return gemm_bf16_run(ctx, desc, a, b, c, bias, aux_in, aux_out, reinterpret_cast<float*>(ctx->workspace),
                       ctx->workspace_bytes, reinterpret_cast<unsigned*>(ctx->gemm_flags));
}
}  // namespace hl

extern "C" int hl_gemm_bf16(hl_ctx* ctx, const hl_gemm_desc* desc, const void* a, const void* b, void* c,
                            const float* bias, const void* aux_in, void* aux_out) {
  return hl::gemm_bf16_ctx(ctx, desc, a, b, c, bias, aux_in, aux_out);
}

extern "C" int hl_gemm_bf16_plan(hl_ctx* ctx, const hl_gemm_desc* desc, int* splits, int* dealt_tiles, size_t* scratch_bytes) {
  if (!ctx || !desc) return hl::fail("hl_gemm_bf16_plan: null argument");
  if (desc->m <= 0 || desc->n <= 0 || desc->k <= 0) return hl::fail("hl_gemm_bf16_plan: m, n, k must be positive");
  const hl::GemmPlan plan = hl::gemm_plan(desc, ctx->sm_count);
  if (splits) *splits = plan.splits;
  if (dealt_tiles) *dealt_tiles = plan.sk_tiles;
  if (scratch_bytes) *scratch_bytes = std::max(plan.splitk_bytes, plan.sk_slot_bytes);
  return HL_OK;
}

// ---- split-K GEMM for callers that must not allocate ----------------------------------------
// hl_gemm_bf16 takes its split-K partial sums from the context's scratch arena and grows that
// arena with the CUDA allocator when a call needs more.  Two kinds of callers of this library
// cannot afford that: a host runtime that has already handed all free device memory to its own
// caching pool (an allocator call there can fail, or succeed only by fragmenting the pool), and
// a step loop whose compute and collective streams are running overlapped, where an allocator
// call may wait for the whole device.  For them the same kernel runs here with its partial sums
// in a fixed array that is part of the library image: every GPU that loads the library holds
// these 32 MiB until the process exits.
namespace hl {
namespace {

constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_gemm_static_scratch[kStaticScratchBytes];
// Flags of the automatic work split (one word per CTA and epilogue warp), apart from the array
// above so that split-K partial sums never land on them.  Static device memory starts at zero and
// launch numbers do not repeat within a process, so a stale flag is never mistaken for a fresh one.
constexpr int kStaticFlagCtas = 256;
static __device__ __align__(256) unsigned g_gemm_static_flags[kStaticFlagCtas * EPI_WARPS];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};  // device address of the array, per device ordinal
void* g_static_flags_addr[kMaxDevices] = {};

// The array's name is only a host-side handle; the address a kernel can use has to be asked for,
// once per device, with that device current.
int static_scratch_address(hl_ctx* ctx, void** out, void** flags_out) {
  HL_REQUIRE(ctx->device >= 0 && ctx->device < kMaxDevices, "hl_gemm_bf16_static_scratch: device ordinal out of range");
  if (g_static_scratch_addr[ctx->device] == nullptr) {
    int current = -1;
    HL_CUDA(cudaGetDevice(&current));
    if (current != ctx->device) HL_CUDA(cudaSetDevice(ctx->device));
    void* ptr = nullptr;
    void* flags = nullptr;
    const cudaError_t e1 = cudaGetSymbolAddress(&ptr, g_gemm_static_scratch);
    const cudaError_t e2 = cudaGetSymbolAddress(&flags, g_gemm_static_flags);
    // the caller's current device is put back before anything is reported
    if (current != ctx->device && current >= 0) HL_CUDA(cudaSetDevice(current));
    HL_CUDA(e1);
    HL_CUDA(e2);
    HL_REQUIRE(ptr != nullptr, "hl_gemm_bf16_static_scratch: the static scratch array has no device address");
    HL_REQUIRE(flags != nullptr, "hl_gemm_bf16_static_scratch: the static flag array has no device address");
    g_static_flags_addr[ctx->device] = flags;
    g_static_scratch_addr[ctx->device] = ptr;
  }
  *out = g_static_scratch_addr[ctx->device];
  *flags_out = g_static_flags_addr[ctx->device];
  return HL_OK;
}

}  // namespace
}  // namespace hl

extern "C" int hl_gemm_bf16_static_scratch(hl_ctx* ctx, const hl_gemm_desc* desc, const void* a, const void* b, void* c,
                                           const float* bias, const void* aux_in, void* aux_out) {
  if (!ctx || !desc) return hl::fail("hl_gemm_bf16_static_scratch: null argument");
  if (ctx->profiler)
    return hl::fail("hl_gemm_bf16_static_scratch: per-kernel timing creates events; turn it off for calls that must not allocate");
  if (desc->m <= 0 || desc->n <= 0 || desc->k <= 0) return hl::fail("hl_gemm_bf16_static_scratch: m, n, k must be positive");
  const hl::GemmPlan plan = hl::gemm_plan(desc, ctx->sm_count);
  const size_t need = std::max(plan.splitk_bytes, plan.sk_slot_bytes);
  if (need > hl::kStaticScratchBytes)
    return hl::fail("hl_gemm_bf16_static_scratch: this shape needs " + std::to_string(need) +
                    " bytes of split-K scratch, more than the fixed " + std::to_string(hl::kStaticScratchBytes) +
                    " bytes; lower split_k or use hl_gemm_bf16");
  if (ctx->sm_count > hl::kStaticFlagCtas)
    return hl::fail("hl_gemm_bf16_static_scratch: more SMs than the fixed flag array covers");
  void* scratch = nullptr;
  void* flags = nullptr;
  int rc = hl::static_scratch_address(ctx, &scratch, &flags);
  if (rc != HL_OK) return rc;
  // Nothing in the scratch array has to start at zero: a launch writes every partial sum that it
  // later reads, so the previous call's contents are simply overwritten.
  return hl::gemm_bf16_run(ctx, desc, a, b, c, bias, aux_in, aux_out, reinterpret_cast<float*>(scratch),
                           hl::kStaticScratchBytes, reinterpret_cast<unsigned*>(flags));
}
