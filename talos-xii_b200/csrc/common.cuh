// Shared host-side plumbing for the talos_b200 library: context, error reporting, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <stdexcept>
#include <string>

#include "../../include/talos_b200.h"

#define TALOS_API extern "C" __attribute__((visibility("default")))

struct talos_error : std::runtime_error {
  talos_status code;
  talos_error(talos_status c, const std::string& m) : std::runtime_error(m), code(c) {}
};

void talos_set_last_error(const std::string& msg);

#define TALOS_CHECK_CUDA(expr)                                                                     \
  do {                                                                                             \
    cudaError_t e__ = (expr);                                                                      \
    if (e__ != cudaSuccess)                                                                        \
      throw talos_error(TALOS_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__));      \
  } while (0)

#define TALOS_REQUIRE(cond, code, msg)                                                             \
  do {                                                                                             \
    if (!(cond)) throw talos_error((code), std::string(msg) + " [" #cond "]");                     \
  } while (0)

// Wraps the body of every extern "C" entry point: exceptions become status codes.
#define TALOS_ENTRY_BEGIN try {
#define TALOS_ENTRY_END                                                                            \
  return TALOS_OK;                                                                                 \
  }                                                                                                \
  catch (const talos_error& e) { talos_set_last_error(e.what()); return e.code; }                  \
  catch (const std::bad_alloc&) { talos_set_last_error("host allocation failed"); return TALOS_ERR_ALLOC; } \
  catch (const std::exception& e) { talos_set_last_error(e.what()); return TALOS_ERR_CUDA; }

struct talos_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = 148;
  void* ws = nullptr;          // kernel-level scratch: split-K partials, column-sum / reduction partials
  size_t ws_bytes = 0;
  void* ws2 = nullptr;         // op-level scratch of composite entry points: dZ of Linear backward, dS of attention
  size_t ws2_bytes = 0;
  int32_t* dev_status = nullptr;   // device-side error word: 1000..2999 a bounded wait gave up, 3000 an index argument was out of range
  int32_t* host_status = nullptr;  // pinned host copy, refreshed by every entry point that blocks on the stream
  int tc_state = 0;            // tensor-core GEMM: 0 = not probed, 1 = active, -1 = disabled
  std::atomic<int64_t> launches{0};
  unsigned dbg_wait_spins = 0;     // test hook (talos_debug_gemm_stall): poll limit of the GEMM kernels' bounded waits, 0 = default
  int dbg_skip_kb = -1;            // test hook: k-block the first CTA's loader leaves out, -1 = none
  struct talos_pool* pool = nullptr;   // caching device allocator behind talos_malloc / talos_free (ctx.cu)
  struct talos_timeline* timeline = nullptr;   // measurement aid (talos_ctx_timeline_begin): one event per launch while recording
};
// Records an event behind the launch just made (ctx.cu); only called while a timeline is being recorded.
void talos_timeline_mark(talos_ctx* ctx, const char* what);

// Device-side error codes written to talos_ctx::dev_status (first writer wins is not required: any non-zero value reports).
#define TALOS_DEV_TIMEOUT_BASE 1000    // + CTA index % 1000 (+ 1000 from the CTA-pair kernel): a bounded mbarrier / flag wait gave up  -> TALOS_ERR_TIMEOUT
#define TALOS_DEV_BAD_INDEX 3000       // an action / index argument read from device memory was out of range -> TALOS_ERR_ARG

// Blocks until the ctx stream is idle, then reports (and clears) the device-side error word: every entry point that
// already waits for the stream calls this instead of cudaStreamSynchronize, so a kernel that gave up is never followed
// by a silent TALOS_OK.
void talos_sync_and_check(talos_ctx* ctx);
// Looks up the device address of talos_colsum_noalloc's fixed scratch array for `device` (which must be current).
void talos_colsum_noalloc_prepare(int device);

// Returns a scratch pointer of at least `bytes`, growing the buffer (stream-ordered free of the
// old one) when needed.
void* talos_workspace(talos_ctx* ctx, size_t bytes);
// Same for the op-level scratch.  Composite entry points use this one so that the kernels they
// call can take their own partial-sum scratch from talos_workspace without overlapping it.
void* talos_workspace2(talos_ctx* ctx, size_t bytes);

inline void talos_check_ctx(talos_ctx* ctx) {
  TALOS_REQUIRE(ctx != nullptr, TALOS_ERR_ARG, "null context");
  TALOS_CHECK_CUDA(cudaSetDevice(ctx->device));
}

// Call after every kernel launch.
inline void talos_launched(talos_ctx* ctx, const char* what) {
  ctx->launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw talos_error(TALOS_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
  if (ctx->timeline) talos_timeline_mark(ctx, what);
}

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- activation helpers shared by the GEMM epilogues and the elementwise kernels ----
// tanh(x) = 1 - 2 / (2^(2x log2 e) + 1) with the hardware exp2 / reciprocal approximations: five dependent
// instructions, no branch, correct limits (+-1) without clamping, |abs error| < 3e-7 (the GEMM epilogues are
// instruction-latency bound, so the short chain matters more than the last bit near zero, where the RELATIVE
// error of this form grows as 1e-7 / |x|).
__device__ __forceinline__ float talos_tanh(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 2.8853900817779268f));   // exp(2x) = 2^(2x log2 e)
  return 1.f - __fdividef(2.f, e + 1.f);                                         // 2/inf = 0 and 2/1 give the +-1 limits
}
__device__ __forceinline__ float talos_act(float v, int act) {
  switch (act) {
    case TALOS_ACT_RELU: return v > 0.f ? v : 0.f;
    case TALOS_ACT_TANH: return talos_tanh(v);
    case TALOS_ACT_SILU: return v / (1.f + __expf(-v));
    default: return v;
  }
}
// Derivative evaluated on the saved tensor: the OUTPUT for relu/tanh, the PRE-activation for silu.
__device__ __forceinline__ float talos_dact(float s, int act) {
  switch (act) {
    case TALOS_ACT_RELU: return s > 0.f ? 1.f : 0.f;
    case TALOS_ACT_TANH: return 1.f - s * s;
    case TALOS_ACT_SILU: { float g = 1.f / (1.f + __expf(-s)); return g * (1.f + s * (1.f - g)); }
    default: return 1.f;
  }
}

// Epilogue in device form (see talos_epilogue in the public header for the order of operations).
struct EpiArgs {
  const float* bias; float* aux_out; long long ld_aux_out; const float* aux_in; long long ld_aux_in;
  int act; int dact; int beta;
};
inline EpiArgs talos_epi_args(const talos_epilogue* e) {
  EpiArgs a{nullptr, nullptr, 0, nullptr, 0, 0, 0, 0};
  if (e) { a.bias = e->bias; a.aux_out = e->aux_out; a.ld_aux_out = e->ld_aux_out; a.aux_in = e->aux_in;
           a.ld_aux_in = e->ld_aux_in; a.act = e->act; a.dact = e->dact; a.beta = e->beta; }
  return a;
}
__device__ __forceinline__ float talos_epilogue_apply(const EpiArgs& e, float acc, long long m, long long n,
                                                      const float* C, long long ldc) {
  float v = acc;
  if (e.bias) v += __ldg(e.bias + n);
  if (e.aux_out) e.aux_out[m * e.ld_aux_out + n] = v;
  if (e.act) v = talos_act(v, e.act);
  if (e.aux_in && e.dact) v *= talos_dact(__ldg(e.aux_in + m * e.ld_aux_in + n), e.dact);
  if (e.beta) v += C[m * ldc + n];
  return v;
}

// Internal cross-file entry points.
void talos_gemm_fp32_launch(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A,
                            int64_t lda, int64_t strideA, const float* B, int64_t ldb, int64_t strideB, float* C,
                            int64_t ldc, int64_t strideC, int64_t batch, const EpiArgs& epi);
// Returns false when the shape/alignment is not eligible (caller falls back to the fp32 kernel).
// First stage of the column sums only: dZ = dY * act'(saved) when dact != 0 (dz may alias dy) and the per-slab column
// sums of dZ left in `partial` ([slabs][n]); returns the slab count, 0 (nothing launched) when the shape is not served.
// The PPO loss kernel without its statistics pass: per-block {loss, kl} sums into partial[blocks][2] (returns blocks =
// ceil(n / 128)) and, when colsum_part is given, per-block column sums of [dlogits | dvalue | 0...] into
// colsum_part[blocks][cs_width] (only where talos_ppo_loss_colsum_supported says so).
int talos_ppo_loss_launch(talos_ctx* ctx, const float* logits, int64_t ld_logits, const float* values, int64_t value_stride, const int32_t* actions,
                          const float* old_logp, const float* adv, const float* ret, int64_t n, int32_t n_actions, float clip, float c_value,
                          float c_entropy, float denom, float* dlogits, int64_t ld_out, float* dvalues, int64_t dvalue_stride, float* partial,
                          float* colsum_part, int cs_width);
bool talos_ppo_loss_colsum_supported(int32_t n_actions, int cs_width);
int talos_colsum_partials_launch(talos_ctx* ctx, const float* dy, float* dz, const float* saved, int dact, int64_t rows, int64_t n,
                                 float* partial, int64_t cap);
// Optional extras for callers that run the same products every step (the PPO trainer):
//  * b_hi / b_lo: the B operand already prepared by the caller with the same shape and pitch as B -- in 3xTF32 mode its
//    TF32 hi / lo split, in TF32 mode b_hi = B rounded to TF32 (b_lo unused) -- so the per-call preparation kernel is
//    skipped (weights change once per optimizer step, not once per product);
//  * partial / partial_floats / splits_out: when the product is split along K, leave the `*splits_out` partial results
//    [splits][M][N] in `partial` (dense, pitch N) and do NOT reduce them into C -- the caller reduces several products'
//    partials in one launch.  *splits_out = 1 means C was written directly (no split, or `partial` too small).
struct TcExtra {
  const float* b_hi = nullptr; const float* b_lo = nullptr;
  float* partial = nullptr; size_t partial_floats = 0; int* splits_out = nullptr;
  // Fused hidden-layer input gradient: C = (A.B^T) * (1 - tanh_saved^2) and per-slab column sums of C into colsum_part
  // ([*colsum_slabs_out][N], summed by the caller).  *colsum_slabs_out stays 0 when the launch did not take the fused
  // route: C is then the plain product and the caller applies the factor itself.
  const float* tanh_saved = nullptr; int64_t ld_saved = 0; float* colsum_part = nullptr; size_t colsum_floats = 0; int* colsum_slabs_out = nullptr;
};
bool talos_gemm_tc_launch(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                          const float* B, int64_t ldb, float* C, int64_t ldc, int mode, const EpiArgs& epi, const TcExtra* extra = nullptr);
// dZ = dY * act'(saved) (dz may alias dy) and db (+)= column sums of dZ in one pass over the rows; false when the
// shape is not served by the vector kernel (n % 4 != 0, n > 1024 or unaligned), in which case nothing was launched.
bool talos_dact_colsum_launch(talos_ctx* ctx, const float* dy, float* dz, const float* saved, int dact, float* db, int64_t rows, int64_t n,
                              int accumulate);
bool talos_gemm_tc_launch_batched(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                                  int64_t strideA, const float* B, int64_t ldb, int64_t strideB, float* C, int64_t ldc, int64_t strideC,
                                  int64_t batch, int mode, const EpiArgs& epi);
