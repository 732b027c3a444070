// fp32 CUDA-core GEMM (FFMA, exact fp32 products): the TALOS_MODE_FP32 arithmetic, the kernel
// for small / skinny / unaligned shapes in every mode, and the on-device check for the
// tensor-core kernel.  NN / NT / TN / TT through element strides, optional batch (grid.z),
// split-K with a deterministic fixed-order reduction, fused epilogue.
#include "common.cuh"

namespace {

struct GemmArgs {
  const float* A; const float* B; float* C;
  long long sAm, sAk, sBk, sBn, ldc;         // element strides of op(A)[m,k], op(B)[k,n]
  long long batchA, batchB, batchC;
  int M, N, K;
  int k_chunk;                                // K range per blockIdx.z slice when split (else K)
  int splits;                                 // >1: write raw partials to `partial`
  float* partial;                             // [splits][M][N]
  EpiArgs epi;
};

// BM x BN tile, BK deep, each thread a TM x TN register block.  Shared tiles are stored
// k-major ([BK][BM], [BK][BN]) so the inner product reads are conflict-free broadcasts.
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_fp32_kernel(GemmArgs g) {
  constexpr int NT = (BM / TM) * (BN / TN);
  __shared__ float As[2][BK][BM + 4];
  __shared__ float Bs[2][BK][BN + 4];

  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  int z = blockIdx.z, batch = 0, kz = 0;
  if (g.splits > 1) kz = z; else batch = z;
  const float* A = g.A + (long long)batch * g.batchA;
  const float* B = g.B + (long long)batch * g.batchB;
  const int k_begin = kz * g.k_chunk;
  const int k_end = min(g.K, k_begin + g.k_chunk);

  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // Loader mapping: walk the contiguous global axis with consecutive threads.
  const bool a_k_contig = (g.sAk == 1);
  const bool b_n_contig = (g.sBn == 1);
  constexpr int A_ELEMS = BM * BK / NT, B_ELEMS = BN * BK / NT;
  static_assert(BM * BK % NT == 0 && BN * BK % NT == 0, "tile/threads mismatch");
  float ra[A_ELEMS], rb[B_ELEMS];

  auto load_tiles = [&](int k0) {
#pragma unroll
    for (int i = 0; i < A_ELEMS; ++i) {
      int e = tid + i * NT, m, k;
      if (a_k_contig) { k = e % BK; m = e / BK; } else { m = e % BM; k = e / BM; }
      int gm = m0 + m, gk = k0 + k;
      ra[i] = (gm < g.M && gk < k_end) ? __ldg(A + (long long)gm * g.sAm + (long long)gk * g.sAk) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < B_ELEMS; ++i) {
      int e = tid + i * NT, n, k;
      if (b_n_contig) { n = e % BN; k = e / BN; } else { k = e % BK; n = e / BK; }
      int gn = n0 + n, gk = k0 + k;
      rb[i] = (gn < g.N && gk < k_end) ? __ldg(B + (long long)gk * g.sBk + (long long)gn * g.sBn) : 0.f;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < A_ELEMS; ++i) {
      int e = tid + i * NT, m, k;
      if (a_k_contig) { k = e % BK; m = e / BK; } else { m = e % BM; k = e / BM; }
      As[buf][k][m] = ra[i];
    }
#pragma unroll
    for (int i = 0; i < B_ELEMS; ++i) {
      int e = tid + i * NT, n, k;
      if (b_n_contig) { n = e % BN; k = e / BN; } else { k = e % BK; n = e / BK; }
      Bs[buf][k][n] = rb[i];
    }
  };

  int buf = 0;
  if (k_begin < k_end) { load_tiles(k_begin); store_tiles(0); }
  __syncthreads();
  for (int k0 = k_begin; k0 < k_end; k0 += BK) {
    const bool more = (k0 + BK) < k_end;
    if (more) load_tiles(k0 + BK);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[buf][k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[buf][k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) { store_tiles(buf ^ 1); }
    __syncthreads();
    buf ^= 1;
  }

  if (g.splits > 1) {
    float* P = g.partial + (long long)kz * g.M * g.N;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      int m = m0 + ty * TM + i; if (m >= g.M) continue;
#pragma unroll
      for (int j = 0; j < TN; ++j) { int n = n0 + tx * TN + j; if (n < g.N) P[(long long)m * g.N + n] = acc[i][j]; }
    }
    return;
  }
  float* C = g.C + (long long)batch * g.batchC;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int m = m0 + ty * TM + i; if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int n = n0 + tx * TN + j; if (n >= g.N) continue;
      C[(long long)m * g.ldc + n] = talos_epilogue_apply(g.epi, acc[i][j], m, n, C, g.ldc);
    }
  }
}

}  // namespace

// Sums `splits` partial [M,N] slabs (deterministic: fixed assignment, fixed order) and applies the
// epilogue.  Scalar version for ragged shapes.
__global__ void talos_splitk_reduce_kernel(const float* __restrict__ partial, int splits, long long M, long long N,
                                           float* C, long long ldc, EpiArgs epi) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * N) return;
  long long m = idx / N, n = idx % N;
  float acc = 0.f;
#pragma unroll 4
  for (int s = 0; s < splits; ++s) acc += __ldcs(partial + (long long)s * M * N + idx);
  C[m * ldc + n] = talos_epilogue_apply(epi, acc, m, n, C, ldc);
}

// Vector version: a CTA covers 64 float4 columns x 4 split lanes; lane l sums slabs l, l+4, ... with
// eight loads in flight, then the four lane sums are added in lane order.
__global__ void __launch_bounds__(256)
talos_splitk_reduce_vec_kernel(const float4* __restrict__ partial, int splits, long long MN4, long long N, float* C,
                               long long ldc, EpiArgs epi) {
  __shared__ float4 sh[4][64];
  const int col = threadIdx.x & 63, sl = threadIdx.x >> 6;
  const long long idx = (long long)blockIdx.x * 64 + col;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (idx < MN4) {
#pragma unroll 8
    for (int s = sl; s < splits; s += 4) {
      const float4 v = __ldcs(partial + (long long)s * MN4 + idx);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  }
  sh[sl][col] = acc;
  __syncthreads();
  if (sl == 0 && idx < MN4) {
    float r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int l = 0; l < 4; ++l) { r[0] += sh[l][col].x; r[1] += sh[l][col].y; r[2] += sh[l][col].z; r[3] += sh[l][col].w; }
    const long long e = idx * 4, m = e / N, n = e % N;          // N % 4 == 0: the four elements share a row
#pragma unroll
    for (int k = 0; k < 4; ++k) C[m * ldc + n + k] = talos_epilogue_apply(epi, r[k], m, n + k, C, ldc);
  }
}

void talos_splitk_reduce(talos_ctx* ctx, const float* partial, int splits, int64_t M, int64_t N, float* C,
                         int64_t ldc, const EpiArgs& epi) {
  int64_t total = M * N;
  if ((N & 3) == 0 && (((uintptr_t)partial) & 15) == 0) {
    talos_splitk_reduce_vec_kernel<<<(unsigned)ceil_div(total / 4, 64), 256, 0, ctx->stream>>>((const float4*)partial, splits, total / 4, N, C, ldc, epi);
  } else {
    talos_splitk_reduce_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, ctx->stream>>>(partial, splits, M, N, C, ldc, epi);
  }
  talos_launched(ctx, "splitk_reduce");
}

void talos_gemm_fp32_launch(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A,
                            int64_t lda, int64_t strideA, const float* B, int64_t ldb, int64_t strideB, float* C,
                            int64_t ldc, int64_t strideC, int64_t batch, const EpiArgs& epi) {
  GemmArgs g;
  g.A = A; g.B = B; g.C = C; g.ldc = ldc;
  g.sAm = opA == TALOS_OP_N ? lda : 1; g.sAk = opA == TALOS_OP_N ? 1 : lda;
  g.sBk = opB == TALOS_OP_N ? ldb : 1; g.sBn = opB == TALOS_OP_N ? 1 : ldb;
  g.batchA = strideA; g.batchB = strideB; g.batchC = strideC;
  g.M = (int)M; g.N = (int)N; g.K = (int)K; g.k_chunk = (int)K; g.splits = 1; g.partial = nullptr; g.epi = epi;

  const bool big = (M >= 96 && N >= 96);
  const int BM = big ? 128 : 64, BN = big ? 128 : 64;
  int64_t tiles = ceil_div(M, BM) * ceil_div(N, BN) * batch;
  // Split the reduction when the output has too few tiles to fill the machine (the dW shape:
  // M,N <= 256 with K = the minibatch).
  int splits = 1;
  if (batch == 1 && tiles * 2 <= ctx->sm_count && K >= 2048) {
    splits = (int)std::min<int64_t>(ceil_div(2 * ctx->sm_count, tiles), K / 512);
    if (splits < 2) splits = 1;
  }
  if (splits > 1) {
    int chunk = (int)ceil_div(K, splits); chunk = (chunk + 15) / 16 * 16;
    splits = (int)ceil_div(K, chunk);
    g.k_chunk = chunk; g.splits = splits;
    g.partial = (float*)talos_workspace(ctx, sizeof(float) * (size_t)splits * M * N);
  }
  dim3 grid((unsigned)ceil_div(N, BN), (unsigned)ceil_div(M, BM), (unsigned)(splits > 1 ? splits : batch));
  if (big) gemm_fp32_kernel<128, 128, 16, 8, 8><<<grid, 256, 0, ctx->stream>>>(g);
  else gemm_fp32_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, ctx->stream>>>(g);
  talos_launched(ctx, "gemm_fp32");
  if (splits > 1) talos_splitk_reduce(ctx, g.partial, splits, M, N, C, ldc, epi);
}

static void check_gemm_args(int32_t opA, int32_t opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                            const float* B, int64_t ldb, float* C, int64_t ldc, int32_t mode) {
  TALOS_REQUIRE((opA == TALOS_OP_N || opA == TALOS_OP_T) && (opB == TALOS_OP_N || opB == TALOS_OP_T), TALOS_ERR_ARG, "bad op");
  TALOS_REQUIRE(mode >= TALOS_MODE_FP32 && mode <= TALOS_MODE_TF32, TALOS_ERR_ARG, "bad mode");
  TALOS_REQUIRE(M >= 0 && N >= 0 && K >= 0 && M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), TALOS_ERR_SHAPE, "bad GEMM extent");
  if (M == 0 || N == 0) return;
  TALOS_REQUIRE(A && B && C, TALOS_ERR_ARG, "null matrix pointer");
  TALOS_REQUIRE(lda >= (opA == TALOS_OP_N ? K : M), TALOS_ERR_SHAPE, "MatMul dimension mismatch: lda too small");
  TALOS_REQUIRE(ldb >= (opB == TALOS_OP_N ? N : K), TALOS_ERR_SHAPE, "MatMul dimension mismatch: ldb too small");
  TALOS_REQUIRE(ldc >= N, TALOS_ERR_SHAPE, "MatMul dimension mismatch: ldc too small");
}

TALOS_API talos_status talos_gemm(talos_ctx* ctx, int32_t opA, int32_t opB, int64_t M, int64_t N, int64_t K,
                                  const float* A, int64_t lda, const float* B, int64_t ldb, float* C, int64_t ldc,
                                  int32_t mode, const talos_epilogue* epi) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  check_gemm_args(opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode);
  if (M == 0 || N == 0) return TALOS_OK;
  EpiArgs e = talos_epi_args(epi);
  TALOS_REQUIRE(!(e.aux_out && e.ld_aux_out < N) && !(e.aux_in && e.ld_aux_in < N), TALOS_ERR_SHAPE, "aux leading dimension too small");
  if (mode != TALOS_MODE_FP32 && talos_gemm_tc_launch(ctx, opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode, e)) return TALOS_OK;
  talos_gemm_fp32_launch(ctx, opA, opB, M, N, K, A, lda, 0, B, ldb, 0, C, ldc, 0, 1, e);
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_gemm_batched(talos_ctx* ctx, int32_t opA, int32_t opB, int64_t M, int64_t N, int64_t K,
                                          const float* A, int64_t lda, int64_t strideA, const float* B, int64_t ldb,
                                          int64_t strideB, float* C, int64_t ldc, int64_t strideC, int64_t batch,
                                          int32_t beta, int32_t mode) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  check_gemm_args(opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode);
  TALOS_REQUIRE(batch >= 0 && batch < 65536 * 16, TALOS_ERR_SHAPE, "bad batch count");
  if (M == 0 || N == 0 || batch == 0) return TALOS_OK;
  EpiArgs e = talos_epi_args(nullptr); e.beta = beta ? 1 : 0;
  if (mode != TALOS_MODE_FP32 &&
      talos_gemm_tc_launch_batched(ctx, opA, opB, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, batch, mode, e))
    return TALOS_OK;
  // grid.z is limited to 65535 slices per launch.
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
    int64_t nb = std::min<int64_t>(65535, batch - b0);
    talos_gemm_fp32_launch(ctx, opA, opB, M, N, K, A + b0 * strideA, lda, strideA, B + b0 * strideB, ldb, strideB,
                           C + b0 * strideC, ldc, strideC, nb, e);
  }
  TALOS_ENTRY_END
}
