// Column sums (the bias gradient, src/autograd.rs:539-543) for callers that must not allocate.
//
// talos_colsum normally takes its partial-sum scratch from the context, which grows it with cudaMalloc
// on demand.  Some callers cannot tolerate that: cudaMalloc synchronises the whole device, so an online
// trainer thread that calls it stalls the kernels of every other thread sharing the GPU (the reference
// runs trainers and simulators side by side, src/main.rs:580-721), and a host that has handed all device
// memory to its own pool may have nothing left for the driver to give.  For them this file keeps the
// scratch in a fixed array that is part of the loaded module: every GPU on which a context is created
// (or this entry point is called) holds these 2 MiB until the process exits.  The array's address is
// resolved when a context is created on the device -- that is when the driver loads the module and sets
// the array aside -- so the calls themselves never allocate or free anything.
#include <mutex>

#include "common.cuh"

namespace {

constexpr int STATIC_MAX_COLS = 1024;       // widest matrix accepted
constexpr int STATIC_MAX_SLABS = 512;       // row slabs summed independently in stage 1
static __device__ __align__(256) float g_colsum_scratch[STATIC_MAX_SLABS * STATIC_MAX_COLS];   // 2 MiB

// In host code the name above is only a handle for the symbol; the kernels need its DEVICE address,
// looked up once per device with that device current.
float* g_scratch_addr[64] = {nullptr};
std::mutex g_scratch_mutex;

float* scratch_for_current_device(int device) {
  TALOS_REQUIRE(device >= 0 && device < 64, TALOS_ERR_ARG, "device index out of range");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[device]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_colsum_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      throw talos_error(TALOS_ERR_CUDA, std::string("cudaGetSymbolAddress(colsum scratch): ") + cudaGetErrorString(e));
    }
    g_scratch_addr[device] = p;
  }
  return g_scratch_addr[device];
}

// Stage 1: CTA `s` sums rows [s*rows_per, (s+1)*rows_per) of every column into scratch[s][*].
__global__ void static_colsum_stage1(const float* __restrict__ g, long long rows, int n, long long rows_per,
                                     float* __restrict__ scratch) {
  const long long r0 = (long long)blockIdx.x * rows_per, r1 = min(rows, r0 + rows_per);
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float s = 0.f;
#pragma unroll 4
    for (long long r = r0; r < r1; ++r) s += g[r * n + c];
    scratch[(size_t)blockIdx.x * n + c] = s;
  }
}
// Stage 2: one thread per column adds the slab sums in slab order.
__global__ void static_colsum_stage2(const float* __restrict__ scratch, int slabs, int n, float* __restrict__ out, int acc) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  float s = 0.f;
  for (int p = 0; p < slabs; ++p) s += scratch[(size_t)p * n + c];
  out[c] = acc ? out[c] + s : s;
}

}  // namespace

// Called by talos_ctx_create with `device` current: the lookup loads this file's module on the device, which is when
// the driver sets the array's 2 MiB aside, so it happens at start-up rather than inside the first call of a thread
// that must not wait for an allocation.  A failure here is not fatal: the entry point repeats the lookup and reports it.
void talos_colsum_noalloc_prepare(int device) {
  try { scratch_for_current_device(device); } catch (const talos_error&) { cudaGetLastError(); }
}

TALOS_API talos_status talos_colsum_noalloc(talos_ctx* ctx, const float* g, float* out, int64_t rows, int64_t n,
                                            int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && n > 0, TALOS_ERR_SHAPE, "bad colsum shape");
  TALOS_REQUIRE(n <= STATIC_MAX_COLS, TALOS_ERR_UNSUPPORTED,
                "talos_colsum_noalloc handles at most 1024 columns (fixed 2 MiB scratch); use talos_colsum for wider matrices");
  TALOS_REQUIRE(g && out, TALOS_ERR_ARG, "null pointer");
  float* scratch = scratch_for_current_device(ctx->device);
  int64_t slabs = std::max<int64_t>(1, std::min<int64_t>(ceil_div(rows, 64), STATIC_MAX_SLABS));
  const int64_t rows_per = std::max<int64_t>(1, ceil_div(rows, slabs));
  slabs = std::max<int64_t>(1, ceil_div(rows, rows_per));
  // Stage 1 overwrites every scratch element stage 2 reads (slabs x n), so nothing left over from an earlier
  // call is ever consumed and nothing needs clearing.
  static_colsum_stage1<<<(unsigned)slabs, 256, 0, ctx->stream>>>(g, rows, (int)n, rows_per, scratch);
  talos_launched(ctx, "colsum_noalloc_stage1");
  static_colsum_stage2<<<(unsigned)ceil_div(n, 128), 128, 0, ctx->stream>>>(scratch, (int)slabs, (int)n, out, accumulate ? 1 : 0);
  talos_launched(ctx, "colsum_noalloc_stage2");
  TALOS_ENTRY_END
}
