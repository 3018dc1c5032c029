// Runtime: contexts, streams, reference-counted buffers, the error channel, device status
// words, counters and TMA tensor-map encoding.  Replaces the Driver-API loader, per-thread
// caches and CudaBuffer machinery of heirloom-kernels/src/cuda.rs:652-949, :7334-7922.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tc05.cuh"

namespace hl {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(const std::string& msg) {
  g_last_error = msg;
  return HL_ERR_INVALID;
}
int fail_cuda(cudaError_t e, const char* what) {
  g_last_error = std::string("CUDA error in ") + what + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
  return HL_ERR_CUDA;
}

int ensure_workspace(hl_ctx* ctx, size_t bytes) {
  if (ctx->workspace_bytes >= bytes) return HL_OK;
  // Grow-only; the old block is released in stream order so kernels still using it finish first.
  if (ctx->workspace) HL_CUDA(cudaFreeAsync(ctx->workspace, ctx->stream));
  ctx->workspace = nullptr;
  ctx->workspace_bytes = 0;
  size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  HL_CUDA(cudaMallocAsync(&ctx->workspace, rounded, ctx->stream));
  ctx->workspace_bytes = rounded;
  ctx->counters.allocations += 1;
  ctx->counters.allocated_bytes += rounded;
  return HL_OK;
}

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                            uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof buf,
             "cuTensorMapEncodeTiled failed (%d): inner=%llu outer=%llu stride=%llu box=%ux%u base=%p", (int)r,
             (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_stride_elems, box_inner,
             box_outer, base);
    return fail(buf);
  }
  return HL_OK;
}

int make_tensor_map(CUtensorMap* out, int dtype, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
  if (swizzle_bytes != 128 && swizzle_bytes != 64 && swizzle_bytes != 32)
    return fail("make_tensor_map: swizzle must be 32, 64 or 128 bytes");
  if (rank < 1 || rank > 5) return fail("make_tensor_map: rank must be in [1, 5]");
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  const CUtensorMapDataType t = dtype == HL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, t, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (%d): rank=%d dims0=%llu dims1=%llu box=%ux%u base=%p", (int)r,
             rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0), box[0], rank > 1 ? box[1] : 0,
             base);
    return fail(buf);
  }
  return HL_OK;
}

int make_tensor_map_bf16_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                            uint64_t stride1_elems, uint64_t stride2_elems, uint32_t box0, uint32_t box1,
                            uint32_t box2) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * 2, stride2_elems * 2};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled (3d) failed (%d): dims=%llu,%llu,%llu box=%u,%u,%u", (int)r,
             (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, box0, box1, box2);
    return fail(buf);
  }
  return HL_OK;
}

struct ProfRecord { cudaEvent_t a, b; int category; double work; };
struct Profiler {
  std::vector<ProfRecord> records;
  std::vector<cudaEvent_t> pool;
  size_t used = 0;
  cudaEvent_t take() {
    if (used == pool.size()) {
      cudaEvent_t e;
      cudaEventCreate(&e);
      pool.push_back(e);
    }
    return pool[used++];
  }
};

void profile_begin(hl_ctx* ctx, int category, double work) {
  Profiler* p = static_cast<Profiler*>(ctx->profiler);
  ProfRecord r{p->take(), p->take(), category, work};
  cudaEventRecord(r.a, ctx->stream);
  p->records.push_back(r);
}
void profile_end(hl_ctx* ctx) {
  Profiler* p = static_cast<Profiler*>(ctx->profiler);
  if (!p->records.empty()) cudaEventRecord(p->records.back().b, ctx->stream);
}

}  // namespace hl

struct hl_buffer {
  hl_ctx* ctx;
  void* ptr;
  size_t bytes;
  std::atomic<int> refs;
};

extern "C" {

const char* hl_last_error(void) { return hl::g_last_error.c_str(); }

unsigned long long hl_fnv1a64(const void* data, size_t bytes, unsigned long long seed) {
  const unsigned char* p = static_cast<const unsigned char*>(data);
  unsigned long long h = seed;
  for (size_t i = 0; i < bytes; ++i) {
    h ^= (unsigned long long)p[i];
    h *= 0x100000001b3ull;
  }
  return h;
}

int hl_ctx_create(int device_ordinal, hl_ctx** out) {
  if (!out) return hl::fail("hl_ctx_create: null output pointer");
  *out = nullptr;
  int count = 0;
  HL_CUDA(cudaGetDeviceCount(&count));
  if (device_ordinal < 0 || device_ordinal >= count)
    return hl::fail("hl_ctx_create: device ordinal " + std::to_string(device_ordinal) + " out of range for " +
                    std::to_string(count) + " devices");
  HL_CUDA(cudaSetDevice(device_ordinal));
  cudaDeviceProp prop;
  HL_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10)
    return hl::fail("hl_ctx_create: this backend is built for sm_100a only; device is sm_" + std::to_string(prop.major) +
                    std::to_string(prop.minor));
  hl_ctx* ctx = new hl_ctx();
  ctx->device = device_ordinal;
  ctx->sm_count = prop.multiProcessorCount;
  HL_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
  HL_CUDA(cudaStreamCreateWithFlags(&ctx->comm_stream, cudaStreamNonBlocking));
  HL_CUDA(cudaMalloc(&ctx->status_dev, sizeof(int) * hl::ST_SLOTS));
  HL_CUDA(cudaMemset(ctx->status_dev, 0, sizeof(int) * hl::ST_SLOTS));
  HL_CUDA(cudaMalloc(&ctx->gemm_sched, 64));
  HL_CUDA(cudaMemset(ctx->gemm_sched, 0, 64));
  HL_CUDA(cudaMallocHost(&ctx->status_host, sizeof(int) * hl::ST_SLOTS));
  memset(ctx->status_host, 0, sizeof(int) * hl::ST_SLOTS);
  *out = ctx;
  return HL_OK;
}

void hl_ctx_destroy(hl_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  cudaStreamSynchronize(ctx->comm_stream);
  if (ctx->profiler) hl_profile_enable(ctx, 0);
  if (ctx->workspace) cudaFree(ctx->workspace);
  if (ctx->gemm_flags) cudaFree(ctx->gemm_flags);
  if (ctx->status_dev) cudaFree(ctx->status_dev);
  if (ctx->gemm_sched) cudaFree(ctx->gemm_sched);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  cudaStreamDestroy(ctx->stream);
  cudaStreamDestroy(ctx->comm_stream);
  delete ctx;
}

int hl_ctx_set_test_hooks(hl_ctx* ctx, unsigned long long wait_limit_ns, int gemm_skip_kblock) {
  HL_REQUIRE(ctx, "hl_ctx_set_test_hooks: null context");
  ctx->wait_limit_ns = wait_limit_ns;
  ctx->gemm_skip_kblock = gemm_skip_kblock;
  return HL_OK;
}

int hl_ctx_sync(hl_ctx* ctx) {
  if (!ctx) return hl::fail("hl_ctx_sync: null context");
  HL_CUDA(cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int) * hl::ST_SLOTS, cudaMemcpyDeviceToHost,
                          ctx->stream));
  HL_CUDA(cudaStreamSynchronize(ctx->stream));
  bool any = false;
  for (int i = 0; i < hl::ST_SLOTS; ++i) any |= ctx->status_host[i] != 0;
  if (any) {
    std::string msg = "device status:";
    if (ctx->status_host[hl::ST_BAD_INDEX]) msg += " out-of-range index (gather/scatter/target);";
    if (ctx->status_host[hl::ST_WAIT_EXPIRED]) msg += " a bounded pipeline wait expired;";
    if (ctx->status_host[hl::ST_BAD_ARGUMENT]) msg += " kernel argument rejected on device;";
    HL_CUDA(cudaMemsetAsync(ctx->status_dev, 0, sizeof(int) * hl::ST_SLOTS, ctx->stream));
    if (ctx->status_host[hl::ST_WAIT_EXPIRED]) {
      // a kernel that gave up did not hand out all of its tiles: the tile counter starts over with the host's copy
      HL_CUDA(cudaMemsetAsync(ctx->gemm_sched, 0, 64, ctx->stream));
      ctx->gemm_sched_base = 0;
    }
    HL_CUDA(cudaStreamSynchronize(ctx->stream));
    hl::set_error(msg);
    return HL_ERR_DEVICE;
  }
  return HL_OK;
}

void* hl_ctx_stream(hl_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int hl_device_info(hl_ctx* ctx, hl_device_info_t* out) {
  if (!ctx || !out) return hl::fail("hl_device_info: null argument");
  cudaDeviceProp prop;
  HL_CUDA(cudaGetDeviceProperties(&prop, ctx->device));
  out->sm_major = prop.major;
  out->sm_minor = prop.minor;
  out->sm_count = prop.multiProcessorCount;
  HL_CUDA(cudaMemGetInfo(&out->free_bytes, &out->total_bytes));
  out->supports_tcgen05 = prop.major == 10 ? 1 : 0;
  return HL_OK;
}

int hl_counters_get(hl_ctx* ctx, hl_counters_t* out) {
  if (!ctx || !out) return hl::fail("hl_counters_get: null argument");
  out->launches = ctx->counters.launches;
  out->gemm_tcgen05_launches = ctx->counters.gemm_tcgen05_launches;
  out->attention_launches = ctx->counters.attention_launches;
  out->h2d_bytes = ctx->counters.h2d_bytes;
  out->d2h_bytes = ctx->counters.d2h_bytes;
  out->allocations = ctx->counters.allocations;
  out->allocated_bytes = ctx->counters.allocated_bytes;
  out->nccl_calls = ctx->counters.nccl_calls;
  out->nccl_bytes = ctx->counters.nccl_bytes;
  out->gemm_pair_launches = ctx->counters.gemm_pair_launches;
  return HL_OK;
}

int hl_counters_reset(hl_ctx* ctx) {
  if (!ctx) return hl::fail("hl_counters_reset: null context");
  ctx->counters = hl::Counters{};
  return HL_OK;
}

int hl_profile_enable(hl_ctx* ctx, int on) {
  if (!ctx) return hl::fail("hl_profile_enable: null context");
  hl::Profiler* p = static_cast<hl::Profiler*>(ctx->profiler);
  if (on) {
    if (!p) ctx->profiler = p = new hl::Profiler();
    p->records.clear();
    p->used = 0;
  } else if (p) {
    HL_CUDA(cudaStreamSynchronize(ctx->stream));
    for (cudaEvent_t e : p->pool) cudaEventDestroy(e);
    delete p;
    ctx->profiler = nullptr;
  }
  return HL_OK;
}

int hl_profile_read(hl_ctx* ctx, hl_profile_t* out) {
  if (!ctx || !out) return hl::fail("hl_profile_read: null argument");
  memset(out, 0, sizeof(*out));
  hl::Profiler* p = static_cast<hl::Profiler*>(ctx->profiler);
  if (!p) return hl::fail("hl_profile_read: profiling is not enabled");
  HL_CUDA(cudaStreamSynchronize(ctx->stream));
  for (const hl::ProfRecord& r : p->records) {
    float ms = 0.f;
    HL_CUDA(cudaEventElapsedTime(&ms, r.a, r.b));
    if (r.category >= 0 && r.category < HL_PROF_CATEGORIES) {
      out->ms[r.category] += ms;
      out->work[r.category] += r.work;
      out->scopes[r.category] += 1;
    }
  }
  p->records.clear();
  p->used = 0;
  return HL_OK;
}

int hl_buffer_alloc(hl_ctx* ctx, size_t bytes, hl_buffer** out) {
  if (!ctx || !out) return hl::fail("hl_buffer_alloc: null argument");
  *out = nullptr;
  void* p = nullptr;
  if (bytes > 0) HL_CUDA(cudaMallocAsync(&p, bytes, ctx->stream));
  hl_buffer* b = new hl_buffer{ctx, p, bytes, {1}};
  ctx->counters.allocations += 1;
  ctx->counters.allocated_bytes += bytes;
  *out = b;
  return HL_OK;
}

int hl_buffer_retain(hl_buffer* buf) {
  if (!buf) return hl::fail("hl_buffer_retain: null buffer");
  buf->refs.fetch_add(1);
  return HL_OK;
}

int hl_buffer_release(hl_buffer* buf) {
  if (!buf) return hl::fail("hl_buffer_release: null buffer");
  if (buf->refs.fetch_sub(1) == 1) {
    // Stream-ordered free: work already queued on the compute stream may still use the block.
    if (buf->ptr) HL_CUDA(cudaFreeAsync(buf->ptr, buf->ctx->stream));
    delete buf;
  }
  return HL_OK;
}

void* hl_buffer_ptr(hl_buffer* buf) { return buf ? buf->ptr : nullptr; }
size_t hl_buffer_bytes(hl_buffer* buf) { return buf ? buf->bytes : 0; }

int hl_memcpy_h2d(hl_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
  if (!ctx || (bytes && (!dst_dev || !src_host))) return hl::fail("hl_memcpy_h2d: null argument");
  HL_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  HL_CUDA(cudaStreamSynchronize(ctx->stream));
  ctx->counters.h2d_bytes += bytes;
  return HL_OK;
}

int hl_memcpy_d2h(hl_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
  if (!ctx || (bytes && (!dst_host || !src_dev))) return hl::fail("hl_memcpy_d2h: null argument");
  HL_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  HL_CUDA(cudaStreamSynchronize(ctx->stream));
  ctx->counters.d2h_bytes += bytes;
  return HL_OK;
}

int hl_memory_copy_indices(hl_ctx* ctx, int64_t* host, const int64_t* dev, long long count) {
  return hl_memcpy_d2h(ctx, host, dev, sizeof(int64_t) * (size_t)count);
}

int hl_memset_zero(hl_ctx* ctx, void* dst_dev, size_t bytes) {
  if (!ctx || (bytes && !dst_dev)) return hl::fail("hl_memset_zero: null argument");
  HL_CUDA(cudaMemsetAsync(dst_dev, 0, bytes, ctx->stream));
  return HL_OK;
}

}  // extern "C"
