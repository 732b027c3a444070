// Linear forward / backward (src/nn.rs:73-133 and the closures it records) as fused GEMM calls.
#include "common.cuh"

namespace {
__global__ void dact_mul_kernel(const float* __restrict__ dy, const float* __restrict__ saved, float* __restrict__ dz,
                                long long n, int act) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dz[i] = dy[i] * talos_dact(saved[i], act);
}
void gemm_any(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
              const float* B, int64_t ldb, float* C, int64_t ldc, int mode, const EpiArgs& e) {
  if (mode != TALOS_MODE_FP32 && talos_gemm_tc_launch(ctx, opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode, e)) return;
  talos_gemm_fp32_launch(ctx, opA, opB, M, N, K, A, lda, 0, B, ldb, 0, C, ldc, 0, 1, e);
}
}  // namespace

TALOS_API talos_status talos_linear_fwd(talos_ctx* ctx, const float* x, const float* W, const float* bias, float* y,
                                        float* z_save, int64_t rows, int64_t in_f, int64_t out_f, int32_t act,
                                        int32_t mode) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && in_f > 0 && out_f > 0, TALOS_ERR_SHAPE, "MatMul dimension mismatch");
  TALOS_REQUIRE(act >= TALOS_ACT_NONE && act <= TALOS_ACT_SILU && mode >= 0 && mode <= TALOS_MODE_TF32, TALOS_ERR_ARG, "bad act/mode");
  if (rows == 0) return TALOS_OK;
  TALOS_REQUIRE(x && W && y, TALOS_ERR_ARG, "null pointer");
  EpiArgs e{bias, z_save, out_f, nullptr, 0, act, 0, 0};
  gemm_any(ctx, TALOS_OP_N, TALOS_OP_N, rows, out_f, in_f, x, in_f, W, out_f, y, out_f, mode, e);
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_linear_bwd(talos_ctx* ctx, const float* x, const float* W, const float* saved,
                                        const float* dy, float* dx, float* dW, float* db, int64_t rows, int64_t in_f,
                                        int64_t out_f, int32_t act, int32_t mode, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && in_f > 0 && out_f > 0, TALOS_ERR_SHAPE, "MatMul dimension mismatch");
  TALOS_REQUIRE(act >= TALOS_ACT_NONE && act <= TALOS_ACT_SILU && mode >= 0 && mode <= TALOS_MODE_TF32, TALOS_ERR_ARG, "bad act/mode");
  if (rows == 0) return TALOS_OK;
  TALOS_REQUIRE(dy && W && (x || !dW), TALOS_ERR_ARG, "null pointer");
  const float* dz = dy;
  bool db_done = false;
  if (act != TALOS_ACT_NONE) {
    TALOS_REQUIRE(saved != nullptr, TALOS_ERR_ARG, "activation backward needs the saved tensor");
    float* buf = (float*)talos_workspace2(ctx, sizeof(float) * (size_t)(rows * out_f));
    // dZ = dY * act'(saved); when the bias gradient is wanted too, the same pass produces its column sums
    if (db && talos_dact_colsum_launch(ctx, dy, buf, saved, act, db, rows, out_f, (accumulate >> 2) & 1)) db_done = true;
    else {
      dact_mul_kernel<<<(unsigned)ceil_div(rows * out_f, 256), 256, 0, ctx->stream>>>(dy, saved, buf, rows * out_f, act);
      talos_launched(ctx, "dact_mul");
    }
    dz = buf;
  }
  if (dx) {   // dL/dx (+)= dZ . W^T   (src/autograd.rs:275-308)
    EpiArgs e{nullptr, nullptr, 0, nullptr, 0, 0, 0, accumulate & 1};
    gemm_any(ctx, TALOS_OP_N, TALOS_OP_T, rows, in_f, out_f, dz, out_f, W, out_f, dx, in_f, mode, e);
  }
  if (dW) {   // dL/dW (+)= x^T . dZ   (src/autograd.rs:310-350)
    EpiArgs e{nullptr, nullptr, 0, nullptr, 0, 0, 0, (accumulate >> 1) & 1};
    gemm_any(ctx, TALOS_OP_T, TALOS_OP_N, in_f, out_f, rows, x, in_f, dz, out_f, dW, out_f, mode, e);
  }
  if (db && !db_done) {   // dL/db (+)= column sums of dZ   (src/autograd.rs:539-543)
    talos_status st = talos_colsum(ctx, dz, db, rows, out_f, (accumulate >> 2) & 1);
    if (st) return st;
  }
  TALOS_ENTRY_END
}
