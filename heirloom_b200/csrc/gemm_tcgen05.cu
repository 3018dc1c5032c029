// bf16 x bf16 -> f32 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory, operands staged by TMA), one persistent warp-specialised kernel family.
//
// Replaces the reference's mma.sync tiers (heirloom-kernels/src/ptx/tensor_core.ptx:42-1527,
// wrappers heirloom-kernels/src/cuda.rs:4215-4386) together with the cast / transpose / pad /
// crop / bias kernels it launches around every matmul (src/nn.rs:432-446,
// src/tensor/autograd.rs:795-850): operand majors are expressed in the TMA descriptors, ragged
// edges by TMA zero fill plus a predicated epilogue, and bias / GELU / residual / dGELU run
// in the epilogue on the f32 accumulators.
//
// Tile: 128 (M) x 256 (N) x 64 (K) per stage, 4 stages (192 KB shared memory), two
// accumulator buffers of 256 tensor-memory columns so the epilogue of tile i overlaps the
// main loop of tile i+1.  Warp roles: warp 0 TMA producer, warp 1 MMA issuer (one elected
// thread), warps 2-5 epilogue (each owns the 32 tensor-memory lanes its warp id maps to).
#include "common.cuh"
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
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr size_t GEMM_SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

struct GemmParams {
  int m, n, k;
  int m_tiles, n_tiles, splits, k_blocks, k_blocks_per_split;
  int epilogue;
  int out_dtype;
  long long ldc;
  long long ld_aux_in;
  long long ld_aux_out;
  void* c;
  const float* bias;
  const void* aux_in;
  void* aux_out;
  float* partials;  // split-K workspace [splits][m][n]
  int* status;
};

struct SharedTail {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedTail* tail = reinterpret_cast<SharedTail*>(smem + size_t(STAGES) * STAGE_BYTES);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_items = p.m_tiles * p.n_tiles * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc05::mbar_init(&tail->full[s], 1);
      tc05::mbar_init(&tail->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc05::mbar_init(&tail->tmem_full[b], 1);
      tc05::mbar_init(&tail->tmem_empty[b], 4);
    }
    tail->abort_flag = 0;
    tc05::fence_barrier_init();
  }
  if (warp == 1) {
    tc05::tmem_alloc(&tail->tmem_base, TMEM_COLS);
    tc05::tmem_relinquish();
  }
  tc05::tc_fence_before_sync();
  __syncthreads();
  tc05::tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (tc05::elect_one()) {
      tc05::tma_prefetch_desc(&map_a);
      tc05::tma_prefetch_desc(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int split = item / (p.m_tiles * p.n_tiles);
        const int rem = item - split * (p.m_tiles * p.n_tiles);
        const int n_tile = rem / p.m_tiles;
        const int m_tile = rem - n_tile * p.m_tiles;
        const int kb0 = split * p.k_blocks_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.k_blocks_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!tc05::mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + size_t(stage) * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          tc05::mbar_arrive_expect_tx(&tail->full[stage], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tc05::tma_load_2d(sa + j * (BK * 128), &map_a, &tail->full[stage], m_tile * BM + j * 64, kb * BK);
          } else {
            tc05::tma_load_2d(sa, &map_a, &tail->full[stage], kb * BK, m_tile * BM);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tc05::tma_load_2d(sb + j * (BK * 128), &map_b, &tail->full[stage], n_tile * BN + j * 64, kb * BK);
          } else {
            tc05::tma_load_2d(sb, &map_b, &tail->full[stage], kb * BK, n_tile * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (tc05::elect_one()) {
      constexpr uint32_t idesc = tc05::instr_desc_bf16_f32(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++local) {
        const int split = item / (p.m_tiles * p.n_tiles);
        const int kb0 = split * p.k_blocks_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.k_blocks_per_split);
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        if (!tc05::mbar_wait(&tail->tmem_empty[buf], buf_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc05::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!tc05::mbar_wait(&tail->full[stage], phase, abort_flag)) { ok = false; break; }
          tc05::tc_fence_after_sync();
          const uint32_t sa = tc05::smem_u32(smem + size_t(stage) * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            const uint64_t da = A_MN ? tc05::smem_desc_sw128(sa + ks * (UMMA_K * 128), BK * 128, 1024)
                                     : tc05::smem_desc_sw128(sa + ks * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? tc05::smem_desc_sw128(sb + ks * (UMMA_K * 128), BK * 128, 1024)
                                     : tc05::smem_desc_sw128(sb + ks * (UMMA_K * 2), 16, 1024);
            tc05::umma_ss(tmem_d, da, db, idesc, (kb > kb0 || ks > 0) ? 1u : 0u);
          }
          tc05::umma_commit(&tail->empty[stage]);  // frees the stage once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc05::umma_commit(&tail->tmem_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..5
    const int lane_group = warp & 3;  // tensor-memory lanes this warp may read
    int local = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++local) {
      const int split = item / (p.m_tiles * p.n_tiles);
      const int rem = item - split * (p.m_tiles * p.n_tiles);
      const int n_tile = rem / p.m_tiles;
      const int m_tile = rem - n_tile * p.m_tiles;
      const int buf = local & 1;
      const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
      if (!tc05::mbar_wait(&tail->tmem_full[buf], buf_phase, abort_flag)) { ok = false; break; }
      tc05::tc_fence_after_sync();
      const int row = m_tile * BM + lane_group * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t taddr_row = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(lane_group * 32) << 16);
#pragma unroll 1
      for (int chunk = 0; chunk < BN / 32; ++chunk) {
        const int col0 = n_tile * BN + chunk * 32;
        if (col0 >= p.n) break;  // uniform across the CTA
        uint32_t acc_bits[32];
        tc05::tmem_ld_32x32b_x32(taddr_row + (uint32_t)(chunk * 32), acc_bits);
        tc05::tmem_ld_wait();
        if (!row_ok) continue;
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(acc_bits[i]);

        if (p.partials != nullptr) {
          float* dst = p.partials + ((size_t)split * p.m + row) * (size_t)p.n + col0;
#pragma unroll
          for (int g = 0; g < 8; ++g)
            if (col0 + g * 4 < p.n)
              *reinterpret_cast<float4*>(dst + g * 4) = make_float4(acc[g * 4], acc[g * 4 + 1], acc[g * 4 + 2], acc[g * 4 + 3]);
          continue;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // groups of 8 columns
          const int col = col0 + g * 8;
          if (col >= p.n) break;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = acc[g * 8 + i];
          if (p.bias != nullptr) {
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + col));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + col + 4));
            v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
            v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
          }
          if (p.epilogue == HL_EPI_BIAS_GELU) {
            // h = bf16(acc + bias) is stored; g = bf16(gelu(h)) goes to aux_out.
            float gl[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { v[i] = bf16_round(v[i]); gl[i] = gelu_fwd_f(v[i]); }
            uint4 o;
            o.x = pack_bf16x2(gl[0], gl[1]); o.y = pack_bf16x2(gl[2], gl[3]);
            o.z = pack_bf16x2(gl[4], gl[5]); o.w = pack_bf16x2(gl[6], gl[7]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.aux_out) + (size_t)row * p.ld_aux_out + col) = o;
          } else if (p.epilogue == HL_EPI_BIAS_RESIDUAL) {
            // out = bf16(residual + bf16(acc + bias)): the two round trips of the block.
            const uint4 r = *reinterpret_cast<const uint4*>(
                reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + (size_t)row * p.ld_aux_in + col);
            const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
            const float rr[8] = {r0.x, r0.y, r1.x, r1.y, r2.x, r2.y, r3.x, r3.y};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = rr[i] + bf16_round(v[i]);
          } else if (p.epilogue == HL_EPI_DGELU) {
            // out = acc * gelu'(h), h read from aux_in.
            const uint4 r = *reinterpret_cast<const uint4*>(
                reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + (size_t)row * p.ld_aux_in + col);
            const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
            const float hh[8] = {r0.x, r0.y, r1.x, r1.y, r2.x, r2.y, r3.x, r3.y};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = v[i] * gelu_grad_f(hh[i]);
          }
          if (p.out_dtype == HL_BF16) {
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.c) + (size_t)row * p.ldc + col) = o;
          } else {
            float* dst = reinterpret_cast<float*>(p.c) + (size_t)row * p.ldc + col;
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
          }
        }
      }
      tc05::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&tail->tmem_empty[buf]);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc05::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // Give copies already in flight time to land before shared memory is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    if (threadIdx.x == 0) atomicExch(p.status + ST_WAIT_EXPIRED, 1);
  }
  if (warp == 1) {
    tc05::tc_fence_after_sync();
    tc05::tmem_dealloc(tmem_base, TMEM_COLS);
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

template <bool A_MN, bool B_MN>
int launch_variant(hl_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int grid) {
  auto kern = gemm_bf16_tcgen05_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    HL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_BYTES));
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, ctx->stream>>>(ma, mb, p);
  HL_LAUNCH_CHECK("gemm_bf16_tcgen05_kernel");
  count_launch(ctx);
  ctx->counters.gemm_tcgen05_launches += 1;
  return HL_OK;
}

}  // namespace

size_t gemm_splitk_workspace_bytes(const hl_gemm_desc* d, int sm_count, int* splits_out) {
  const int m_tiles = ceil_div(d->m, BM), n_tiles = ceil_div(d->n, BN);
  const int k_blocks = ceil_div(d->k, BK);
  int splits = d->split_k;
  if (splits <= 0) {
    splits = 1;
    if (d->epilogue == HL_EPI_NONE && d->out_dtype == HL_F32) {
      // Fill the machine when the output has few tiles and the contraction is long.
      const int tiles = m_tiles * n_tiles;
      if (tiles < sm_count && k_blocks >= 16) splits = min(min(sm_count / tiles, k_blocks / 8), 32);
      if (splits < 1) splits = 1;
    }
  }
  splits = min(splits, k_blocks);
  int per = ceil_div(k_blocks, splits);
  splits = ceil_div(k_blocks, per);  // every split owns at least one k block
  if (splits_out) *splits_out = splits;
  return splits > 1 ? (size_t)splits * d->m * (size_t)d->n * sizeof(float) : 0;
}

int gemm_bf16_run(hl_ctx* ctx, const hl_gemm_desc* d, const void* a, const void* b, void* c, const float* bias,
                  const void* aux_in, void* aux_out, float* workspace, size_t workspace_bytes) {
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
  HL_REQUIRE(d->lda >= (a_mn ? d->m : d->k) && d->ldb >= (b_mn ? d->n : d->k) && d->ldc >= d->n,
             "hl_gemm_bf16: leading dimension smaller than the row length");
  switch (d->epilogue) {
    case HL_EPI_NONE: break;
    case HL_EPI_BIAS: HL_REQUIRE(bias, "hl_gemm_bf16: bias epilogue needs a bias"); break;
    case HL_EPI_BIAS_GELU:
      HL_REQUIRE(bias && aux_out && d->out_dtype == HL_BF16, "hl_gemm_bf16: bias+gelu needs bias, aux_out and bf16 output");
      break;
    case HL_EPI_BIAS_RESIDUAL:
      HL_REQUIRE(bias && aux_in && d->out_dtype == HL_BF16, "hl_gemm_bf16: bias+residual needs bias, aux_in and bf16 output");
      break;
    case HL_EPI_DGELU: HL_REQUIRE(aux_in, "hl_gemm_bf16: dgelu epilogue needs aux_in"); break;
    default: return fail("hl_gemm_bf16: unknown epilogue");
  }
  if (bias) HL_REQUIRE((reinterpret_cast<uintptr_t>(bias) & 15) == 0, "hl_gemm_bf16: bias must be 16-byte aligned");

  GemmParams p{};
  p.m = d->m; p.n = d->n; p.k = d->k;
  p.m_tiles = ceil_div(d->m, BM);
  p.n_tiles = ceil_div(d->n, BN);
  p.k_blocks = ceil_div(d->k, BK);
  int splits = 1;
  const size_t need = gemm_splitk_workspace_bytes(d, ctx->sm_count, &splits);
  p.splits = splits;
  p.k_blocks_per_split = ceil_div(p.k_blocks, splits);
  p.epilogue = d->epilogue;
  p.out_dtype = d->out_dtype;
  p.ldc = d->ldc;
  p.ld_aux_in = d->ld_aux_in > 0 ? d->ld_aux_in : d->ldc;
  p.ld_aux_out = d->ld_aux_out > 0 ? d->ld_aux_out : d->ldc;
  p.c = c; p.bias = bias; p.aux_in = aux_in; p.aux_out = aux_out;
  p.status = ctx->status_dev;
  p.partials = nullptr;
  if (splits > 1) {
    HL_REQUIRE(d->epilogue == HL_EPI_NONE && d->out_dtype == HL_F32, "hl_gemm_bf16: split-K needs a plain f32 output");
    HL_REQUIRE(d->n % 4 == 0, "hl_gemm_bf16: split-K needs n % 4 == 0");
    HL_REQUIRE(workspace != nullptr && workspace_bytes >= need, "hl_gemm_bf16: split-K scratch is too small");
    p.partials = workspace;
  }

  CUtensorMap ma, mb;
  int rc;
  if (a_mn) rc = make_tensor_map_bf16_2d(&ma, a, (uint64_t)d->m, (uint64_t)d->k, (uint64_t)d->lda, 64, BK);
  else      rc = make_tensor_map_bf16_2d(&ma, a, (uint64_t)d->k, (uint64_t)d->m, (uint64_t)d->lda, BK, BM);
  if (rc != HL_OK) return rc;
  if (b_mn) rc = make_tensor_map_bf16_2d(&mb, b, (uint64_t)d->n, (uint64_t)d->k, (uint64_t)d->ldb, 64, BK);
  else      rc = make_tensor_map_bf16_2d(&mb, b, (uint64_t)d->k, (uint64_t)d->n, (uint64_t)d->ldb, BK, BN);
  if (rc != HL_OK) return rc;

  const int total = p.m_tiles * p.n_tiles * p.splits;
  const int grid = min(total, ctx->sm_count);
  ProfileScope prof(ctx, HL_PROF_GEMM, 2.0 * (double)d->m * (double)d->n * (double)d->k);
  if (a_mn && b_mn) rc = launch_variant<true, true>(ctx, ma, mb, p, grid);
  else if (a_mn)    rc = launch_variant<true, false>(ctx, ma, mb, p, grid);
  else if (b_mn)    rc = launch_variant<false, true>(ctx, ma, mb, p, grid);
  else              rc = launch_variant<false, false>(ctx, ma, mb, p, grid);
  if (rc != HL_OK) return rc;
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

extern "C" int hl_gemm_bf16(hl_ctx* ctx, const hl_gemm_desc* desc, const void* a, const void* b, void* c,
                            const float* bias, const void* aux_in, void* aux_out) {
  if (!ctx || !desc) return hl::fail("hl_gemm_bf16: null argument");
  const size_t need = hl::gemm_splitk_workspace_bytes(desc, ctx->sm_count, nullptr);
  if (need > 0) {
    int rc = hl::ensure_workspace(ctx, need);
    if (rc != HL_OK) return rc;
  }
  return hl::gemm_bf16_run(ctx, desc, a, b, c, bias, aux_in, aux_out, reinterpret_cast<float*>(ctx->workspace),
                           ctx->workspace_bytes);
}
