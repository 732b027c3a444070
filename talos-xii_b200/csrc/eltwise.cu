// Layout ops (transpose, concat/split, last_token, bias broadcast) and the elementwise /
// reduction ops of the autograd engine.
#include "common.cuh"

namespace {

struct TransposeArgs { long long in_stride[6]; long long out_shape[6]; int rank; };

// General axis swap.  Each thread produces one output element; when the innermost axis is
// untouched the innermost index is contiguous on both sides, so loads and stores coalesce.
__global__ void transpose_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, TransposeArgs a, int acc) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  long long rem = idx, src = 0;
#pragma unroll
  for (int d = 5; d >= 0; --d) {
    if (d < a.rank) { long long c = rem % a.out_shape[d]; rem /= a.out_shape[d]; src += c * a.in_stride[d]; }
  }
  float v = x[src];
  y[idx] = acc ? y[idx] + v : v;
}

// 2-D tiled transpose of the two innermost axes ([batch, R, C] -> [batch, C, R]) through shared memory.
__global__ void transpose2d_kernel(const float* __restrict__ x, float* __restrict__ y, int R, int Cc, int acc) {
  __shared__ float tile[32][33];
  const float* xb = x + (long long)blockIdx.z * R * Cc; float* yb = y + (long long)blockIdx.z * R * Cc;
  int c = blockIdx.x * 32 + threadIdx.x, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) { int r = r0 + i; if (r < R && c < Cc) tile[i][threadIdx.x] = xb[(long long)r * Cc + c]; }
  __syncthreads();
  int r = r0 + threadIdx.x, c0 = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int cc = c0 + i;
    if (r < R && cc < Cc) { long long o = (long long)cc * R + r; float v = tile[threadIdx.x][i]; yb[o] = acc ? yb[o] + v : v; }
  }
}

__global__ void concat_last_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                   long long rows, int da, int db) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int w = da + db; if (idx >= rows * w) return;
  long long r = idx / w; int c = (int)(idx % w);
  out[idx] = c < da ? a[r * da + c] : b[r * db + (c - da)];
}
__global__ void split_last_kernel(const float* __restrict__ g, float* __restrict__ ga, float* __restrict__ gb,
                                  long long rows, int da, int db, int acc) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int w = da + db; if (idx >= rows * w) return;
  long long r = idx / w; int c = (int)(idx % w); float v = g[idx];
  if (c < da) { if (ga) { long long o = r * da + c; ga[o] = acc ? ga[o] + v : v; } }
  else if (gb) { long long o = r * db + (c - da); gb[o] = acc ? gb[o] + v : v; }
}
__global__ void last_token_kernel(const float* __restrict__ x, float* __restrict__ y, long long B, long long S, int D) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * D) return;
  long long b = idx / D; int d = (int)(idx % D);
  y[idx] = x[(b * S + (S - 1)) * D + d];
}
__global__ void bias_add_kernel(float* __restrict__ y, const float* __restrict__ bias, long long total, int n) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) y[idx] += __ldg(bias + (idx % n));
}

__device__ __forceinline__ float ew_fwd(int op, float x, float p0, float p1) {
  switch (op) {
    case TALOS_EW_RELU: return x > 0.f ? x : 0.f;
    case TALOS_EW_TANH: return tanhf(x);
    case TALOS_EW_SILU: return x / (1.f + expf(-x));
    case TALOS_EW_EXP: return expf(x);
    case TALOS_EW_LOG: return logf(x);
    case TALOS_EW_SIN: return sinf(x);
    case TALOS_EW_COS: return cosf(x);
    case TALOS_EW_SQRT: return sqrtf(x);
    case TALOS_EW_CLIP: return fminf(fmaxf(x, p0), p1);
    case TALOS_EW_NEG: return -x;
    case TALOS_EW_SCALE: return x * p0;
    default: return x;
  }
}
// Derivative on the INPUT x, as the reference's closures compute it (src/autograd.rs:370-382,
// :399-409, :426-437, :560-570, :587-597, :614-626, :752-764; scale: src/transformer.rs:1063-1068).
__device__ __forceinline__ float ew_bwd(int op, float x, float p0, float p1) {
  switch (op) {
    case TALOS_EW_RELU: return x > 0.f ? 1.f : 0.f;
    case TALOS_EW_TANH: { float t = tanhf(x); return 1.f - t * t; }
    case TALOS_EW_SILU: { float s = 1.f / (1.f + expf(-x)); return s * (1.f + x * (1.f - s)); }
    case TALOS_EW_EXP: return expf(x);
    case TALOS_EW_LOG: return 1.f / x;
    case TALOS_EW_SIN: return cosf(x);
    case TALOS_EW_COS: return -sinf(x);
    case TALOS_EW_SQRT: return x > 0.f ? 0.5f / sqrtf(x) : 0.f;
    case TALOS_EW_CLIP: return (x >= p0 && x <= p1) ? 1.f : 0.f;       // inclusive bounds
    case TALOS_EW_NEG: return -1.f;
    case TALOS_EW_SCALE: return p0;
    default: return 1.f;
  }
}
__global__ void ew_unary_kernel(int op, const float* __restrict__ x, float* __restrict__ y, long long n, float p0, float p1) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = ew_fwd(op, x[i], p0, p1);
}
__global__ void ew_unary_bwd_kernel(int op, const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx,
                                    long long n, float p0, float p1) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dx[i] += dy[i] * ew_bwd(op, x[i], p0, p1);
}
__global__ void ew_binary_kernel(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, long long n) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float u = a[i], v = b[i];
  y[i] = op == TALOS_EW_ADD ? u + v : op == TALOS_EW_SUB ? u - v : op == TALOS_EW_MUL ? u * v : u / v;
}
// da/db may alias (x op x): both contributions are then added by the same thread in turn.
__global__ void ew_binary_bwd_kernel(int op, const float* a, const float* b, const float* __restrict__ dy, float* da, float* db, long long n) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float g = dy[i], u = a[i], v = b[i], ga, gb;
  switch (op) {
    case TALOS_EW_ADD: ga = g; gb = g; break;
    case TALOS_EW_SUB: ga = g; gb = -g; break;
    case TALOS_EW_MUL: ga = g * v; gb = g * u; break;
    default: ga = g / v; gb = -g * u / (v * v); break;
  }
  if (da) da[i] += ga;
  if (db) db[i] += gb;
}

// Deterministic sum: fixed grid, fixed per-thread order, second stage sums block partials in order.
__global__ void reduce_stage1_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float sh[256];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) s += x[i];
  sh[threadIdx.x] = s; __syncthreads();
  for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o]; __syncthreads(); }
  if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
__global__ void reduce_stage2_kernel(const float* __restrict__ partial, int nparts, float scale, float* out, int acc) {
  __shared__ float sh[256];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 256) s += partial[i];
  sh[threadIdx.x] = s; __syncthreads();
  for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o]; __syncthreads(); }
  if (threadIdx.x == 0) out[0] = acc ? out[0] + sh[0] * scale : sh[0] * scale;
}
__global__ void fill_from_scalar_kernel(const float* __restrict__ s, float scale, float* __restrict__ y, long long n, int acc) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { float v = s[0] * scale; y[i] = acc ? y[i] + v : v; }
}

inline unsigned blocks_for(int64_t n) { return (unsigned)ceil_div(n, 256); }

}  // namespace

TALOS_API talos_status talos_transpose(talos_ctx* ctx, const float* x, float* y, const int64_t* shape, int32_t rank,
                                       int32_t d0, int32_t d1, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(shape && rank >= 1 && rank <= 6 && d0 >= 0 && d1 >= 0 && d0 < rank && d1 < rank, TALOS_ERR_SHAPE, "bad transpose axes");
  int64_t n = 1; for (int i = 0; i < rank; ++i) { TALOS_REQUIRE(shape[i] >= 0, TALOS_ERR_SHAPE, "negative extent"); n *= shape[i]; }
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(x && y, TALOS_ERR_ARG, "null pointer");
  int lo = std::min(d0, d1), hi = std::max(d0, d1);
  if (hi == rank - 1 && lo == rank - 2 && lo != hi) {
    int64_t batch = n / (shape[lo] * shape[hi]);
    if (batch <= 65535) {
      dim3 grid((unsigned)ceil_div(shape[hi], 32), (unsigned)ceil_div(shape[lo], 32), (unsigned)batch);
      transpose2d_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(x, y, (int)shape[lo], (int)shape[hi], accumulate ? 1 : 0);
      talos_launched(ctx, "transpose2d");
      return TALOS_OK;
    }
  }
  TransposeArgs a; a.rank = rank;
  long long in_stride[6], st = 1;
  for (int i = rank - 1; i >= 0; --i) { in_stride[i] = st; st *= shape[i]; }
  for (int i = 0; i < rank; ++i) { a.out_shape[i] = shape[i]; a.in_stride[i] = in_stride[i]; }
  std::swap(a.out_shape[d0], a.out_shape[d1]); std::swap(a.in_stride[d0], a.in_stride[d1]);
  for (int i = rank; i < 6; ++i) { a.out_shape[i] = 1; a.in_stride[i] = 0; }
  transpose_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(x, y, n, a, accumulate ? 1 : 0);
  talos_launched(ctx, "transpose");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_concat_last(talos_ctx* ctx, const float* a, const float* b, float* out, int64_t rows, int64_t da, int64_t db) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && da >= 0 && db >= 0 && da + db < (1 << 30), TALOS_ERR_SHAPE, "bad concat shape");
  int64_t n = rows * (da + db); if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(a && b && out, TALOS_ERR_ARG, "null pointer");
  concat_last_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(a, b, out, rows, (int)da, (int)db);
  talos_launched(ctx, "concat_last");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_split_last(talos_ctx* ctx, const float* g, float* ga, float* gb, int64_t rows, int64_t da, int64_t db, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && da >= 0 && db >= 0 && da + db < (1 << 30), TALOS_ERR_SHAPE, "bad split shape");
  int64_t n = rows * (da + db); if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(g, TALOS_ERR_ARG, "null pointer");
  split_last_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(g, ga, gb, rows, (int)da, (int)db, accumulate ? 1 : 0);
  talos_launched(ctx, "split_last");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_last_token(talos_ctx* ctx, const float* x, float* y, int64_t B, int64_t S, int64_t D) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(B >= 0 && S >= 1 && D >= 0 && D < (1 << 30), TALOS_ERR_SHAPE, "bad last_token shape");
  if (B * D == 0) return TALOS_OK;
  TALOS_REQUIRE(x && y, TALOS_ERR_ARG, "null pointer");
  last_token_kernel<<<blocks_for(B * D), 256, 0, ctx->stream>>>(x, y, B, S, (int)D);
  talos_launched(ctx, "last_token");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_bias_add(talos_ctx* ctx, float* y, const float* bias, int64_t rows, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && n > 0 && n < (1 << 30), TALOS_ERR_SHAPE, "Add shape mismatch");
  if (rows == 0) return TALOS_OK;
  TALOS_REQUIRE(y && bias, TALOS_ERR_ARG, "null pointer");
  bias_add_kernel<<<blocks_for(rows * n), 256, 0, ctx->stream>>>(y, bias, rows * n, (int)n);
  talos_launched(ctx, "bias_add");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_eltwise_unary(talos_ctx* ctx, int32_t op, const float* x, float* y, int64_t n, float p0, float p1) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(op >= TALOS_EW_RELU && op <= TALOS_EW_SCALE, TALOS_ERR_ARG, "bad unary op");
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "negative length"); if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(x && y, TALOS_ERR_ARG, "null pointer");
  ew_unary_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(op, x, y, n, p0, p1);
  talos_launched(ctx, "eltwise_unary");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_eltwise_unary_bwd(talos_ctx* ctx, int32_t op, const float* x, const float* dy, float* dx, int64_t n, float p0, float p1) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(op >= TALOS_EW_RELU && op <= TALOS_EW_SCALE, TALOS_ERR_ARG, "bad unary op");
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "negative length"); if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(x && dy && dx, TALOS_ERR_ARG, "null pointer");
  ew_unary_bwd_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(op, x, dy, dx, n, p0, p1);
  talos_launched(ctx, "eltwise_unary_bwd");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_eltwise_binary(talos_ctx* ctx, int32_t op, const float* a, const float* b, float* y, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(op >= TALOS_EW_ADD && op <= TALOS_EW_DIV, TALOS_ERR_ARG, "bad binary op");
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "negative length"); if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(a && b && y, TALOS_ERR_ARG, "null pointer");
  ew_binary_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(op, a, b, y, n);
  talos_launched(ctx, "eltwise_binary");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_eltwise_binary_bwd(talos_ctx* ctx, int32_t op, const float* a, const float* b, const float* dy, float* da, float* db, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(op >= TALOS_EW_ADD && op <= TALOS_EW_DIV, TALOS_ERR_ARG, "bad binary op");
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "negative length"); if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(a && b && dy, TALOS_ERR_ARG, "null pointer");
  ew_binary_bwd_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(op, a, b, dy, da, db, n);
  talos_launched(ctx, "eltwise_binary_bwd");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_reduce_sum(talos_ctx* ctx, const float* x, int64_t n, float scale, float* out, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "negative length");
  TALOS_REQUIRE(out && (x || n == 0), TALOS_ERR_ARG, "null pointer");
  int parts = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n, 1024), 1024));
  float* partial = (float*)talos_workspace(ctx, sizeof(float) * parts);
  reduce_stage1_kernel<<<parts, 256, 0, ctx->stream>>>(x, n, partial);
  talos_launched(ctx, "reduce_stage1");
  reduce_stage2_kernel<<<1, 256, 0, ctx->stream>>>(partial, parts, scale, out, accumulate ? 1 : 0);
  talos_launched(ctx, "reduce_stage2");
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_fill_from_scalar(talos_ctx* ctx, const float* s, float scale, float* y, int64_t n, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "negative length"); if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(s && y, TALOS_ERR_ARG, "null pointer");
  fill_from_scalar_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(s, scale, y, n, accumulate ? 1 : 0);
  talos_launched(ctx, "fill_from_scalar");
  TALOS_ENTRY_END
}
