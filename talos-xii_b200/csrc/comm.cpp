// Gradient exchange over NCCL (NVLink 5 / NVSwitch).  NCCL is bound at run time with dlopen so the
// library has no link-time dependency on it: inside a process that already carries an NCCL (for
// example torch's) that instance is reused, otherwise the system libnccl.so.2 is loaded.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "../../include/talos_b200_ppo.h"

namespace {
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
constexpr int kNcclFloat32 = 7, kNcclSum = 0;

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
    api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
    api.CommAbort = (decltype(api.CommAbort))dlsym(h, "ncclCommAbort");
    api.CommGetAsyncError = (decltype(api.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
    api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy && api.GetErrorString;
  });
  return api;
}

void nccl_check(ncclResult_t r, const char* what) {
  if (r != 0) throw talos_error(TALOS_ERR_NCCL, std::string(what) + ": " + (nccl().GetErrorString ? nccl().GetErrorString(r) : "NCCL error"));
}
}  // namespace

struct talos_comm { talos_ctx* ctx; ncclComm_t comm; int nranks, rank; };

TALOS_API talos_status talos_comm_unique_id(uint8_t* id_out) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(id_out != nullptr, TALOS_ERR_ARG, "null id buffer");
  TALOS_REQUIRE(nccl().ok, TALOS_ERR_NCCL, "libnccl.so.2 could not be loaded");
  ncclUniqueId id; nccl_check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
  memcpy(id_out, id.internal, 128);
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_comm_init(talos_ctx* ctx, const uint8_t* id_host, int32_t nranks, int32_t rank, talos_comm** out) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(id_host && out, TALOS_ERR_ARG, "null pointer");
  TALOS_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, TALOS_ERR_ARG, "bad rank / world size");
  TALOS_REQUIRE(nccl().ok, TALOS_ERR_NCCL, "libnccl.so.2 could not be loaded");
  ncclUniqueId id; memcpy(id.internal, id_host, 128);
  ncclComm_t c = nullptr;
  nccl_check(nccl().CommInitRank(&c, nranks, id, rank), "ncclCommInitRank");
  *out = new talos_comm{ctx, c, nranks, rank};
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_comm_destroy(talos_comm* comm) {
  TALOS_ENTRY_BEGIN
  if (!comm) return TALOS_OK;
  cudaSetDevice(comm->ctx->device);
  cudaStreamSynchronize(comm->ctx->stream);
  if (comm->comm) nccl().CommDestroy(comm->comm);
  delete comm;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_comm_allreduce_sum(talos_comm* comm, float* buf, int64_t n) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(comm != nullptr, TALOS_ERR_ARG, "null communicator");
  talos_check_ctx(comm->ctx);
  TALOS_REQUIRE(n >= 0 && (buf || n == 0), TALOS_ERR_ARG, "bad buffer");
  if (n == 0) return TALOS_OK;
  if (nccl().CommGetAsyncError) {   // a rank that died shows up here before the next collective is enqueued
    ncclResult_t async = 0;
    nccl_check(nccl().CommGetAsyncError(comm->comm, &async), "ncclCommGetAsyncError");
    nccl_check(async, "NCCL asynchronous error");
  }
  nccl_check(nccl().AllReduce(buf, buf, (size_t)n, kNcclFloat32, kNcclSum, comm->comm, comm->ctx->stream), "ncclAllReduce");
  comm->ctx->launches.fetch_add(1, std::memory_order_relaxed);
  TALOS_ENTRY_END
}
