// NCCL binding for the data-parallel gradient exchange.  The library is opened at run time
// ("libnccl.so.2", or the path in HEIRLOOM_NCCL_LIB) like the reference does
// (heirloom-kernels/src/cuda.rs:7954-8307: unique id, init_rank, all_reduce_sum_in_place_f32,
// abort), so the backend has no link-time dependency on NCCL.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <algorithm>

#include "kernels.h"

namespace hl {
namespace {

typedef struct { char internal[128]; } NcclUniqueId;
typedef void* NcclComm;
constexpr int kNcclFloat32 = 7;
constexpr int kNcclUint8 = 1;
constexpr int kNcclSum = 0;
constexpr int kNcclMax = 2;

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*CommAbort)(NcclComm) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*GetVersion)(int*) = nullptr;
};

NcclApi* api() {
  static NcclApi a;
  static bool tried = false;
  if (tried) return a.handle ? &a : nullptr;
  tried = true;
  const char* path = getenv("HEIRLOOM_NCCL_LIB");
  a.handle = dlopen(path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!a.handle) return nullptr;
#define HL_SYM(field, name)                                              \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.handle, name)); \
  if (!a.field) { a.handle = nullptr; return nullptr; }
  HL_SYM(GetUniqueId, "ncclGetUniqueId")
  HL_SYM(CommInitRank, "ncclCommInitRank")
  HL_SYM(AllReduce, "ncclAllReduce")
  HL_SYM(CommDestroy, "ncclCommDestroy")
  HL_SYM(CommAbort, "ncclCommAbort")
  HL_SYM(GetErrorString, "ncclGetErrorString")
  HL_SYM(GetVersion, "ncclGetVersion")
#undef HL_SYM
  return &a;
}

struct NcclState {
  NcclComm comm = nullptr;
  int rank = 0, world = 1;
};

int fail_nccl(int code, const char* what) {
  NcclApi* a = api();
  set_error(std::string("NCCL error in ") + what + ": " + (a ? a->GetErrorString(code) : "library not loaded"));
  return HL_ERR_NCCL;
}

}  // namespace

bool nccl_active(const hl_ctx* ctx) { return ctx->nccl != nullptr && static_cast<NcclState*>(ctx->nccl)->world > 1; }
int nccl_world(const hl_ctx* ctx) { return ctx->nccl ? static_cast<NcclState*>(ctx->nccl)->world : 1; }

int nccl_allreduce_sum_f32(hl_ctx* ctx, float* buf, size_t count, cudaStream_t stream) {
  NcclState* st = static_cast<NcclState*>(ctx->nccl);
  HL_REQUIRE(st && st->comm, "NCCL communicator is not initialised");
  int rc = api()->AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, st->comm, stream);
  if (rc != 0) return fail_nccl(rc, "ncclAllReduce");
  ctx->counters.nccl_calls += 1;
  ctx->counters.nccl_bytes += count * sizeof(float);
  return HL_OK;
}

// Element-wise maximum of a byte mask over the ranks: the union of the rows any rank selected
// (the reference's sparse data-parallel exchange, src/bin/heirloom/runtime.rs:4171-4214).
int nccl_allreduce_max_u8(hl_ctx* ctx, unsigned char* buf, size_t count, cudaStream_t stream) {
  NcclState* st = static_cast<NcclState*>(ctx->nccl);
  HL_REQUIRE(st && st->comm, "NCCL communicator is not initialised");
  int rc = api()->AllReduce(buf, buf, count, kNcclUint8, kNcclMax, st->comm, stream);
  if (rc != 0) return fail_nccl(rc, "ncclAllReduce");
  ctx->counters.nccl_calls += 1;
  ctx->counters.nccl_bytes += count;
  return HL_OK;
}

}  // namespace hl

using namespace hl;

extern "C" {

int hl_nccl_version(int* out) {
  HL_REQUIRE(out, "hl_nccl_version: null argument");
  NcclApi* a = api();
  if (!a) { set_error(std::string("cannot load NCCL: ") + (dlerror() ? dlerror() : "libnccl.so.2 not found")); return HL_ERR_NCCL; }
  int rc = a->GetVersion(out);
  return rc == 0 ? HL_OK : fail_nccl(rc, "ncclGetVersion");
}

int hl_nccl_unique_id(unsigned char out[128]) {
  HL_REQUIRE(out, "hl_nccl_unique_id: null argument");
  NcclApi* a = api();
  if (!a) { set_error("cannot load NCCL (libnccl.so.2)"); return HL_ERR_NCCL; }
  NcclUniqueId id;
  int rc = a->GetUniqueId(&id);
  if (rc != 0) return fail_nccl(rc, "ncclGetUniqueId");
  memcpy(out, id.internal, 128);
  return HL_OK;
}

int hl_nccl_init(hl_ctx* ctx, int rank, int world, const unsigned char id_bytes[128]) {
  HL_REQUIRE(ctx && id_bytes, "hl_nccl_init: null argument");
  HL_REQUIRE(world >= 1 && rank >= 0 && rank < world, "hl_nccl_init: rank must be in [0, world)");
  HL_REQUIRE(ctx->nccl == nullptr, "hl_nccl_init: communicator already initialised");
  NcclApi* a = api();
  if (!a) { set_error("cannot load NCCL (libnccl.so.2)"); return HL_ERR_NCCL; }
  HL_CUDA(cudaSetDevice(ctx->device));
  NcclUniqueId id;
  memcpy(id.internal, id_bytes, 128);
  NcclState* st = new NcclState();
  st->rank = rank;
  st->world = world;
  // HEIRLOOM_COMM_SMS=R gives the collective kernels at most R SMs and makes the persistent GEMM / attention kernels
  // leave exactly those free while collectives are in flight; the default, 0, leaves NCCL its own choice and reserves
  // nothing (at 8 GPUs: 21.84 ms a step against 22.07 with R = 8 and 21.97 with R = 16, where the capped collectives
  // finish later than the backward pass they hide behind).  NCCL reads its bound from the environment when the
  // communicator is made; a value the user set is kept.
  int comm_sms = 0;
  if (const char* e = getenv("HEIRLOOM_COMM_SMS")) comm_sms = std::max(0, std::min(atoi(e), ctx->sm_count / 2));
  if (world > 1 && comm_sms > 0) {
    const std::string v = std::to_string(comm_sms);
    setenv("NCCL_MAX_CTAS", v.c_str(), 0);
    ctx->comm_sms = comm_sms;
  }
  int rc = a->CommInitRank(&st->comm, world, id, rank);
  if (rc != 0) { delete st; return fail_nccl(rc, "ncclCommInitRank"); }
  ctx->nccl = st;
  return HL_OK;
}

int hl_nccl_allreduce_f32(hl_ctx* ctx, float* buf_dev, size_t count) {
  HL_REQUIRE(ctx && (buf_dev || count == 0), "hl_nccl_allreduce_f32: null argument");
  if (count == 0) return HL_OK;
  // Ordered after the compute stream's queued work and before its later work, like the
  // reference's blocking in-place all-reduce (cuda.rs:8159-8206) but without a host sync.
  return nccl_allreduce_sum_f32(ctx, buf_dev, count, ctx->stream);
}

int hl_nccl_allreduce_max_u8(hl_ctx* ctx, unsigned char* buf_dev, size_t count) {
  HL_REQUIRE(ctx && (buf_dev || count == 0), "hl_nccl_allreduce_max_u8: null argument");
  if (count == 0) return HL_OK;
  return nccl_allreduce_max_u8(ctx, buf_dev, count, ctx->stream);
}

int hl_nccl_abort(hl_ctx* ctx) {
  HL_REQUIRE(ctx, "hl_nccl_abort: null context");
  NcclState* st = static_cast<NcclState*>(ctx->nccl);
  if (!st) return HL_OK;
  if (st->comm) api()->CommAbort(st->comm);
  delete st;
  ctx->nccl = nullptr;
  ctx->comm_sms = ctx->reserve_sms = 0;
  return HL_OK;
}

int hl_nccl_destroy(hl_ctx* ctx) {
  HL_REQUIRE(ctx, "hl_nccl_destroy: null context");
  NcclState* st = static_cast<NcclState*>(ctx->nccl);
  if (!st) return HL_OK;
  if (st->comm) api()->CommDestroy(st->comm);
  delete st;
  ctx->nccl = nullptr;
  ctx->comm_sms = ctx->reserve_sms = 0;
  return HL_OK;
}

}  // extern "C"
