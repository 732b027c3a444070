// The slice primitives of src/simd.rs as callable device ops: add_scaled_row (:2-32), dot_product (:34-63),
// vector_fma (:66-94), softmax_exp_sum (:333-359) and vector_scale (:362-379).  The crate calls them on short f64
// slices from Linear::forward_inference and both batched matmuls; here each is one launch over a device vector of any
// length (128-bit accesses when the pointers allow it, a scalar tail otherwise), HBM-bound: 12 / 8 / 16 / 8 / 8 bytes
// per element.  Reductions are two-stage with a fixed combination order, so results are reproducible run to run.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int MAX_BLOCKS = 1024;

__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x < 32) {
    t = threadIdx.x < (THREADS >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  __syncthreads();
  return t;                                            // valid in warp 0
}
__device__ __forceinline__ float block_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -INFINITY;
  if (threadIdx.x < 32) {
    t = threadIdx.x < (THREADS >> 5) ? sh[threadIdx.x] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  }
  __syncthreads();
  return t;
}

// kind 0: out += scale * a (add_scaled_row); 1: out += a * b (vector_fma); 2: out *= scale (vector_scale)
template <int KIND>
__global__ void __launch_bounds__(THREADS)
axpy_like_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, float scale, long long n, int vec) {
  const long long tid = (long long)blockIdx.x * THREADS + threadIdx.x, nthreads = (long long)gridDim.x * THREADS;
  long long done = 0;
  if (vec) {
    const long long n4 = n >> 2;
    for (long long i = tid; i < n4; i += nthreads) {
      float4 o = ((float4*)out)[i];
      if (KIND == 0) { const float4 x = __ldg((const float4*)a + i); o.x += scale * x.x; o.y += scale * x.y; o.z += scale * x.z; o.w += scale * x.w; }
      if (KIND == 1) {
        const float4 x = __ldg((const float4*)a + i), y = __ldg((const float4*)b + i);
        o.x += x.x * y.x; o.y += x.y * y.y; o.z += x.z * y.z; o.w += x.w * y.w;
      }
      if (KIND == 2) { o.x *= scale; o.y *= scale; o.z *= scale; o.w *= scale; }
      ((float4*)out)[i] = o;
    }
    done = n4 << 2;
  }
  for (long long i = done + tid; i < n; i += nthreads) {
    if (KIND == 0) out[i] += scale * a[i];
    if (KIND == 1) out[i] += a[i] * b[i];
    if (KIND == 2) out[i] *= scale;
  }
}

__global__ void __launch_bounds__(THREADS)
dot_stage1_kernel(const float* __restrict__ a, const float* __restrict__ b, long long n, int vec, float* __restrict__ partial) {
  __shared__ float sh[THREADS / 32];
  const long long tid = (long long)blockIdx.x * THREADS + threadIdx.x, nthreads = (long long)gridDim.x * THREADS;
  float s = 0.f; long long done = 0;
  if (vec) {
    const long long n4 = n >> 2;
    for (long long i = tid; i < n4; i += nthreads) {
      const float4 x = __ldg((const float4*)a + i), y = __ldg((const float4*)b + i);
      s += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
    }
    done = n4 << 2;
  }
  for (long long i = done + tid; i < n; i += nthreads) s += a[i] * b[i];
  s = block_sum(s, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// One block adds the stage-1 partials (strided, then the fixed shuffle tree) and writes / accumulates the scalar.
__global__ void __launch_bounds__(THREADS)
sum_partials_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out, int accumulate) {
  __shared__ float sh[THREADS / 32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += THREADS) s += partial[i];
  s = block_sum(s, sh);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

__global__ void __launch_bounds__(THREADS)
max_stage1_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float sh[THREADS / 32];
  float m = -INFINITY;
  for (long long i = (long long)blockIdx.x * THREADS + threadIdx.x; i < n; i += (long long)gridDim.x * THREADS) m = fmaxf(m, x[i]);
  m = block_max(m, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = m;
}
// row[i] = exp(row[i] - max); per-block sums of the results.  Every block first reduces the (few) per-block maxima.
__global__ void __launch_bounds__(THREADS)
exp_sum_stage2_kernel(float* __restrict__ x, long long n, const float* __restrict__ max_partial, int nparts, float* __restrict__ sum_partial) {
  __shared__ float sh[THREADS / 32];
  __shared__ float mx_s;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < nparts; i += THREADS) m = fmaxf(m, max_partial[i]);
  m = block_max(m, sh);
  if (threadIdx.x == 0) mx_s = m;
  __syncthreads();
  const float mx = mx_s;
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * THREADS + threadIdx.x; i < n; i += (long long)gridDim.x * THREADS) {
    const float e = expf(x[i] - mx); x[i] = e; s += e;
  }
  s = block_sum(s, sh);
  if (threadIdx.x == 0) sum_partial[blockIdx.x] = s;
}

int blocks_for(talos_ctx* ctx, int64_t n, int per_thread) {
  return (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n, (int64_t)THREADS * per_thread), std::min(MAX_BLOCKS, 8 * ctx->sm_count)));
}
bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr) {
  return ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c)) & 15) == 0;
}

}  // namespace

TALOS_API talos_status talos_axpy(talos_ctx* ctx, float* out, const float* row, float scale, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "Dimension mismatch in add_scaled_row");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(out && row, TALOS_ERR_ARG, "null pointer");
  axpy_like_kernel<0><<<blocks_for(ctx, n, 8), THREADS, 0, ctx->stream>>>(out, row, nullptr, scale, n, aligned16(out, row) ? 1 : 0);
  talos_launched(ctx, "axpy");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_vector_fma(talos_ctx* ctx, float* dst, const float* a, const float* b, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "bad length");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(dst && a && b, TALOS_ERR_ARG, "null pointer");
  axpy_like_kernel<1><<<blocks_for(ctx, n, 8), THREADS, 0, ctx->stream>>>(dst, a, b, 0.f, n, aligned16(dst, a, b) ? 1 : 0);
  talos_launched(ctx, "vector_fma");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_vector_scale(talos_ctx* ctx, float* row, float scale, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "bad length");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(row != nullptr, TALOS_ERR_ARG, "null pointer");
  axpy_like_kernel<2><<<blocks_for(ctx, n, 8), THREADS, 0, ctx->stream>>>(row, nullptr, nullptr, scale, n, aligned16(row) ? 1 : 0);
  talos_launched(ctx, "vector_scale");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_dot(talos_ctx* ctx, const float* a, const float* b, int64_t n, float* out, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "Dimension mismatch in dot_product");
  TALOS_REQUIRE(out != nullptr && ((a && b) || n == 0), TALOS_ERR_ARG, "null pointer");
  const int blocks = blocks_for(ctx, n, 16);
  float* partial = (float*)talos_workspace(ctx, sizeof(float) * MAX_BLOCKS);
  dot_stage1_kernel<<<blocks, THREADS, 0, ctx->stream>>>(a, b, n, aligned16(a, b) ? 1 : 0, partial);
  talos_launched(ctx, "dot_stage1");
  sum_partials_kernel<<<1, THREADS, 0, ctx->stream>>>(partial, blocks, out, accumulate ? 1 : 0);
  talos_launched(ctx, "dot_stage2");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_softmax_exp_sum(talos_ctx* ctx, float* row, int64_t n, float* sum_out) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "bad length");
  TALOS_REQUIRE(sum_out != nullptr && (row || n == 0), TALOS_ERR_ARG, "null pointer");
  if (n == 0) { TALOS_CHECK_CUDA(cudaMemsetAsync(sum_out, 0, sizeof(float), ctx->stream)); return TALOS_OK; }   // empty row: 0.0 (:336-338)
  const int blocks = blocks_for(ctx, n, 8);
  float* partial = (float*)talos_workspace(ctx, sizeof(float) * 2 * MAX_BLOCKS);
  max_stage1_kernel<<<blocks, THREADS, 0, ctx->stream>>>(row, n, partial);
  talos_launched(ctx, "exp_sum_max");
  exp_sum_stage2_kernel<<<blocks, THREADS, 0, ctx->stream>>>(row, n, partial, blocks, partial + MAX_BLOCKS);
  talos_launched(ctx, "exp_sum_exp");
  sum_partials_kernel<<<1, THREADS, 0, ctx->stream>>>(partial + MAX_BLOCKS, blocks, sum_out, 0);
  talos_launched(ctx, "exp_sum_sum");
  TALOS_ENTRY_END
}
