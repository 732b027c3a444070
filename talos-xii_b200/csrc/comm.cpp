// Gradient exchange over NCCL (NVLink 5 / NVSwitch).  NCCL is bound at run time with dlopen so the
// library has no link-time dependency on it: inside a process that already carries an NCCL (for
// example torch's) that instance is reused, otherwise the system libnccl.so.2 is loaded.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "comm.cuh"

namespace {
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
constexpr int kNcclFloat32 = 7, kNcclSum = 0;

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
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
    api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
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

namespace {
constexpr int kNcclInt8 = 0;
constexpr size_t XCHG_SLOT_FLOATS = size_t(1) << 20;          // 4 MiB per slot: 1 M gradient floats per exchange

// Maps every rank's exchange area into this process (CUDA IPC; the handles travel through an NCCL all-gather).  Any
// failure on any rank leaves the peer-memory path off on ALL ranks (they agree through an all-reduce), and the NCCL
// all-reduce keeps serving the exchange.
void setup_peer_exchange(talos_comm* c) {
  talos_xchg& x = c->x;
  if (c->nranks < 2 || c->nranks > TALOS_MAX_RANKS || getenv("TALOS_COMM_NO_P2P") || !nccl().AllGather) return;
  cudaStream_t st = c->ctx->stream; ncclComm_t nc = (ncclComm_t)c->nccl;
  const size_t bytes = 1024 + 2 * XCHG_SLOT_FLOATS * sizeof(float);
  char* area = nullptr; char* hbuf = nullptr; float* okbuf = nullptr;
  bool ok = cudaMalloc(&area, bytes) == cudaSuccess && cudaMalloc(&hbuf, (size_t)c->nranks * sizeof(cudaIpcMemHandle_t)) == cudaSuccess &&
            cudaMalloc(&okbuf, sizeof(float)) == cudaSuccess;
  cudaIpcMemHandle_t mine; memset(&mine, 0, sizeof(mine));
  if (ok) ok = cudaMemsetAsync(area, 0, bytes, st) == cudaSuccess && cudaIpcGetMemHandle(&mine, area) == cudaSuccess;
  std::string all((size_t)c->nranks * sizeof(cudaIpcMemHandle_t), '\0');
  if (ok) {                                                    // (a rank that failed so far cannot take part in the gather: see the agreement below)
    ok = cudaMemcpyAsync(hbuf + (size_t)c->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice, st) == cudaSuccess &&
         nccl().AllGather(hbuf + (size_t)c->rank * sizeof(mine), hbuf, sizeof(mine), kNcclInt8, nc, st) == 0 &&
         cudaMemcpyAsync(&all[0], hbuf, all.size(), cudaMemcpyDeviceToHost, st) == cudaSuccess && cudaStreamSynchronize(st) == cudaSuccess;
  }
  if (ok) {
    for (int r = 0; r < c->nranks && ok; ++r) {
      if (r == c->rank) { x.peer[r] = area; continue; }
      cudaIpcMemHandle_t h; memcpy(&h, &all[(size_t)r * sizeof(h)], sizeof(h));
      void* p = nullptr;
      ok = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
      x.peer[r] = (char*)p;
    }
  }
  cudaGetLastError();
  // agreement: the path is on only if it is on everywhere
  float mine_ok = ok ? 1.f : 0.f, total = 0.f;
  bool agreed = okbuf && cudaMemcpyAsync(okbuf, &mine_ok, sizeof(float), cudaMemcpyHostToDevice, st) == cudaSuccess &&
                nccl().AllReduce(okbuf, okbuf, 1, kNcclFloat32, kNcclSum, nc, st) == 0 &&
                cudaMemcpyAsync(&total, okbuf, sizeof(float), cudaMemcpyDeviceToHost, st) == cudaSuccess && cudaStreamSynchronize(st) == cudaSuccess;
  cudaFree(hbuf); cudaFree(okbuf);
  if (agreed && total == (float)c->nranks) { x.active = true; x.local = area; x.slot_floats = XCHG_SLOT_FLOATS; return; }
  for (int r = 0; r < c->nranks; ++r) { if (r != c->rank && x.peer[r]) cudaIpcCloseMemHandle(x.peer[r]); x.peer[r] = nullptr; }
  cudaFree(area); cudaGetLastError();
}

void teardown_peer_exchange(talos_comm* c) {
  talos_xchg& x = c->x;
  if (!x.active) return;
  // nobody may still be reading this rank's area: one last collective after the stream has drained
  float* okbuf = nullptr;
  if (cudaMalloc(&okbuf, sizeof(float)) == cudaSuccess) {
    cudaMemsetAsync(okbuf, 0, sizeof(float), c->ctx->stream);
    nccl().AllReduce(okbuf, okbuf, 1, kNcclFloat32, kNcclSum, (ncclComm_t)c->nccl, c->ctx->stream);
    cudaStreamSynchronize(c->ctx->stream);
    cudaFree(okbuf);
  }
  for (int r = 0; r < c->nranks; ++r) if (r != c->rank && x.peer[r]) cudaIpcCloseMemHandle(x.peer[r]);
  cudaFree(x.local);
  x.active = false; cudaGetLastError();
}
}  // namespace

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
  talos_comm* cm = new talos_comm{ctx, (void*)c, nranks, rank, talos_xchg{}};
  setup_peer_exchange(cm);
  *out = cm;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_comm_destroy(talos_comm* comm) {
  TALOS_ENTRY_BEGIN
  if (!comm) return TALOS_OK;
  cudaSetDevice(comm->ctx->device);
  cudaStreamSynchronize(comm->ctx->stream);
  teardown_peer_exchange(comm);
  if (comm->nccl) nccl().CommDestroy((ncclComm_t)comm->nccl);
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
    nccl_check(nccl().CommGetAsyncError((ncclComm_t)comm->nccl, &async), "ncclCommGetAsyncError");
    nccl_check(async, "NCCL asynchronous error");
  }
  nccl_check(nccl().AllReduce(buf, buf, (size_t)n, kNcclFloat32, kNcclSum, (ncclComm_t)comm->nccl, comm->ctx->stream), "ncclAllReduce");
  comm->ctx->launches.fetch_add(1, std::memory_order_relaxed);
  TALOS_ENTRY_END
}

TALOS_API int32_t talos_comm_peer_exchange_active(talos_comm* comm) { return comm && comm->x.active ? 1 : 0; }

TALOS_API talos_status talos_debug_comm_stall(talos_comm* comm, int32_t skip_next_signal, uint32_t wait_spins) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(comm != nullptr, TALOS_ERR_ARG, "null communicator");
  TALOS_REQUIRE(wait_spins == 0 || wait_spins >= 1024, TALOS_ERR_ARG, "bad poll limit");
  comm->x.dbg_skip_signal = skip_next_signal ? 1 : 0; comm->x.wait_spins = wait_spins;
  TALOS_ENTRY_END
}
