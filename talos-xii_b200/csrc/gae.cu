// Advantage estimation on the device (src/ppo.rs:650-675): reward normalisation clipped to +-10, the reverse GAE
// recurrence over the whole rollout buffer, and the advantage normalisation (mean, population std + 1e-8).
//
// The recurrence gae[t] = b[t] + a[t] * gae[t+1] (a = gamma*lambda*nonterminal, b = delta) is a chain of affine maps,
// and affine maps compose associatively, so it runs as a three-pass scan: every block folds its 2 048 elements into
// one map, one thread chains the block maps from the end of the buffer, every block replays its elements from its
// carry-in.  The result does not depend on the launch geometry beyond fp32 rounding of the composed maps.
#include "common.cuh"

namespace {

constexpr int GAE_THREADS = 256, GAE_PER_THREAD = 8, GAE_CHUNK = GAE_THREADS * GAE_PER_THREAD;

struct Affine { float a, b; };                                            // x -> a*x + b
__device__ __forceinline__ Affine compose(Affine outer, Affine inner) { return Affine{outer.a * inner.a, fmaf(outer.a, inner.b, outer.b)}; }

struct GaeArgs {
  const float* rewards; const float* values; const int32_t* terminals; long long len;
  float gamma, gl, rew_mean, rew_inv_std;
};

// a[t], b[t] of one element (src/ppo.rs:654-665) from its reward, value, next value and terminal flag.
__device__ __forceinline__ Affine gae_element(const GaeArgs& g, float reward, float v, float vn, int terminal) {
  float r = (reward - g.rew_mean) * g.rew_inv_std;
  r = fminf(fmaxf(r, -10.f), 10.f);
  const float nt = terminal ? 0.f : 1.f;
  return Affine{g.gl * nt, r + g.gamma * vn * nt - v};
}

// The 8 consecutive elements a thread owns, in registers: 128-bit loads when the whole group is inside the buffer and
// the arrays are 16-byte aligned (a warp then reads 1 KB of each array contiguously), element-wise otherwise.
struct GaeGroup { float r[GAE_PER_THREAD], v[GAE_PER_THREAD + 1]; int term[GAE_PER_THREAD]; int count; };
__device__ __forceinline__ void gae_load(const GaeArgs& g, long long t0, bool aligned, GaeGroup& e) {
  e.count = (int)max(0LL, min((long long)GAE_PER_THREAD, g.len - t0));
  if (aligned && e.count == GAE_PER_THREAD) {
    const float4 r0 = *(const float4*)(g.rewards + t0), r1 = *(const float4*)(g.rewards + t0 + 4);
    const float4 v0 = *(const float4*)(g.values + t0), v1 = *(const float4*)(g.values + t0 + 4);
    const int4 m0 = *(const int4*)(g.terminals + t0), m1 = *(const int4*)(g.terminals + t0 + 4);
    e.r[0] = r0.x; e.r[1] = r0.y; e.r[2] = r0.z; e.r[3] = r0.w; e.r[4] = r1.x; e.r[5] = r1.y; e.r[6] = r1.z; e.r[7] = r1.w;
    e.v[0] = v0.x; e.v[1] = v0.y; e.v[2] = v0.z; e.v[3] = v0.w; e.v[4] = v1.x; e.v[5] = v1.y; e.v[6] = v1.z; e.v[7] = v1.w;
    e.term[0] = m0.x; e.term[1] = m0.y; e.term[2] = m0.z; e.term[3] = m0.w; e.term[4] = m1.x; e.term[5] = m1.y; e.term[6] = m1.z; e.term[7] = m1.w;
  } else {
#pragma unroll
    for (int i = 0; i < GAE_PER_THREAD; ++i) {
      const bool in = i < e.count;
      e.r[i] = in ? g.rewards[t0 + i] : 0.f; e.v[i] = in ? g.values[t0 + i] : 0.f; e.term[i] = in ? g.terminals[t0 + i] : 1;
    }
  }
  e.v[GAE_PER_THREAD] = (t0 + GAE_PER_THREAD < g.len) ? g.values[t0 + GAE_PER_THREAD] : 0.f;     // V[len] = 0 (src/ppo.rs:662)
}

// PASS 0: block_maps[blk] = composition of the block's elements (first element outermost).
// PASS 1: replay with the carry-in carries[blk] = gae just past the block's last element; write advantages / returns.
template <int PASS>
__global__ void __launch_bounds__(GAE_THREADS)
gae_scan_kernel(GaeArgs g, int aligned, Affine* block_maps, const float* __restrict__ carries, float* __restrict__ advantages, float* __restrict__ returns) {
  __shared__ Affine warp_maps[GAE_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long t0 = (long long)blockIdx.x * GAE_CHUNK + (long long)tid * GAE_PER_THREAD;
  GaeGroup e;
  gae_load(g, t0, aligned != 0, e);
  // this thread's own map: its elements folded from the last one inwards
  Affine mine{1.f, 0.f};
#pragma unroll
  for (int i = GAE_PER_THREAD - 1; i >= 0; --i) if (i < e.count) mine = compose(gae_element(g, e.r[i], e.v[i], e.v[i + 1], e.term[i]), mine);
  // suffix scan over the threads of the block: after[tid] = map of all elements of the block behind this thread's
  Affine incl = mine;                                                       // inclusive suffix within the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    Affine other{__shfl_down_sync(0xffffffffu, incl.a, o), __shfl_down_sync(0xffffffffu, incl.b, o)};
    if (lane + o < 32) incl = compose(incl, other);
  }
  if (lane == 0) warp_maps[warp] = incl;
  __syncthreads();
  Affine behind_warps{1.f, 0.f};                                            // maps of the warps behind this one
  for (int w = GAE_THREADS / 32 - 1; w > warp; --w) behind_warps = compose(warp_maps[w], behind_warps);
  Affine excl{__shfl_down_sync(0xffffffffu, incl.a, 1), __shfl_down_sync(0xffffffffu, incl.b, 1)};
  if (lane == 31) excl = Affine{1.f, 0.f};
  const Affine after = compose(excl, behind_warps);
  if (PASS == 0) {
    if (tid == 0) block_maps[blockIdx.x] = compose(mine, after);
  } else {
    float gae = fmaf(after.a, carries[blockIdx.x], after.b);                // value entering this thread's last element
    float adv[GAE_PER_THREAD];
#pragma unroll
    for (int i = GAE_PER_THREAD - 1; i >= 0; --i) {
      if (i < e.count) { const Affine m = gae_element(g, e.r[i], e.v[i], e.v[i + 1], e.term[i]); gae = fmaf(m.a, gae, m.b); }
      adv[i] = gae;
    }
    if (aligned && e.count == GAE_PER_THREAD) {
      *(float4*)(advantages + t0) = make_float4(adv[0], adv[1], adv[2], adv[3]);
      *(float4*)(advantages + t0 + 4) = make_float4(adv[4], adv[5], adv[6], adv[7]);
      *(float4*)(returns + t0) = make_float4(adv[0] + e.v[0], adv[1] + e.v[1], adv[2] + e.v[2], adv[3] + e.v[3]);
      *(float4*)(returns + t0 + 4) = make_float4(adv[4] + e.v[4], adv[5] + e.v[5], adv[6] + e.v[6], adv[7] + e.v[7]);
    } else {
#pragma unroll
      for (int i = 0; i < GAE_PER_THREAD; ++i) if (i < e.count) { advantages[t0 + i] = adv[i]; returns[t0 + i] = adv[i] + e.v[i]; }
    }
  }
}

// carries[blk] = gae just past block blk's last element; the buffer ends with gae = 0 (src/ppo.rs:651).  One block:
// each thread folds a run of consecutive block maps, the runs are suffix-scanned in shared memory, each thread
// replays its run.
constexpr int CHAIN_THREADS = 1024;
__global__ void __launch_bounds__(CHAIN_THREADS)
gae_chain_kernel(const Affine* __restrict__ block_maps, float* __restrict__ carries, int blocks) {
  __shared__ Affine sh[CHAIN_THREADS];
  const int tid = threadIdx.x, per = (blocks + CHAIN_THREADS - 1) / CHAIN_THREADS;
  const int b0 = tid * per, b1 = min(blocks, b0 + per);
  Affine mine{1.f, 0.f};
  for (int b = b1 - 1; b >= b0; --b) mine = compose(block_maps[b], mine);
  sh[tid] = mine;
  __syncthreads();
  for (int o = 1; o < CHAIN_THREADS; o <<= 1) {                           // inclusive suffix scan of the runs
    Affine other{1.f, 0.f};
    if (tid + o < CHAIN_THREADS) other = sh[tid + o];
    __syncthreads();
    sh[tid] = compose(sh[tid], other);
    __syncthreads();
  }
  float x = (tid + 1 < CHAIN_THREADS) ? sh[tid + 1].b : 0.f;              // the runs behind this one, applied to gae = 0
  for (int b = b1 - 1; b >= b0; --b) { carries[b] = x; x = fmaf(block_maps[b].a, x, block_maps[b].b); }
}

// ---- advantage normalisation: two deterministic two-stage reductions and one elementwise pass --------------------------
constexpr int RED_THREADS = 256;
__device__ __forceinline__ double block_sum(double v, double* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  double s = 0.0;
  if (threadIdx.x == 0) for (int w = 0; w < RED_THREADS / 32; ++w) s += sh[w];
  return s;                                                                 // valid in thread 0
}
// SQDIFF 0: partial sums of x;  1: partial sums of (x - stats[0])^2.  VEC: x is 16-byte aligned (n4 = n / 4 groups).
template <int SQDIFF>
__global__ void __launch_bounds__(RED_THREADS)
moment_partial_kernel(const float* __restrict__ x, long long n, int vec, const float* __restrict__ stats, double* __restrict__ partials) {
  __shared__ double sh[RED_THREADS / 32];
  const float mean = SQDIFF ? stats[0] : 0.f;
  const long long stride = (long long)gridDim.x * RED_THREADS, first = (long long)blockIdx.x * RED_THREADS + threadIdx.x;
  double acc = 0.0;
  auto term = [&](float v) { const float d = v - mean; return SQDIFF ? (double)d * d : (double)d; };
  const long long n4 = vec ? n / 4 : 0;
  for (long long i = first; i < n4; i += stride) {
    const float4 v = __ldg((const float4*)x + i);
    acc += (term(v.x) + term(v.y)) + (term(v.z) + term(v.w));
  }
  for (long long i = 4 * n4 + first; i < n; i += stride) acc += term(x[i]);
  const double s = block_sum(acc, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}
// stats[0] = mean (SQDIFF 0)  or  stats[1] = sqrt(sum / n) + 1e-8 (SQDIFF 1).  One block: thread t adds partials
// t, t + 256, ... and thread 0 adds the 256 thread sums in thread order -- a fixed order, so the result is reproducible
// (a single thread walking all partials took 49 us for 1 184 of them: one dependent L2 load each).
template <int SQDIFF>
__global__ void __launch_bounds__(RED_THREADS)
moment_final_kernel(const double* __restrict__ partials, int count, long long n, float* stats) {
  __shared__ double sh[RED_THREADS];
  double acc = 0.0;
  for (int i = threadIdx.x; i < count; i += RED_THREADS) acc += partials[i];
  sh[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x != 0) return;
  double s = 0.0;
  for (int i = 0; i < RED_THREADS; ++i) s += sh[i];
  if (SQDIFF) stats[1] = (float)(sqrt(s / (double)n) + 1e-8); else stats[0] = (float)(s / (double)n);
}
__global__ void normalize_kernel(const float* x, long long n, int vec, const float* __restrict__ stats, float* y) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const float mean = stats[0], sd = stats[1];
  if (vec) {
    if (4 * i + 3 < n) {
      float4 v = *((const float4*)x + i);
      v.x = (v.x - mean) / sd; v.y = (v.y - mean) / sd; v.z = (v.z - mean) / sd; v.w = (v.w - mean) / sd;
      *((float4*)y + i) = v;
    } else {
      for (long long j = 4 * i; j < n; ++j) y[j] = (x[j] - mean) / sd;
    }
  } else if (i < n) {
    y[i] = (x[i] - mean) / sd;
  }
}

}  // namespace

TALOS_API talos_status talos_gae(talos_ctx* ctx, const float* rewards, const float* values, const int32_t* terminals, int64_t len,
                                 float gamma, float lambda, float rew_mean, float rew_var, float* advantages, float* returns) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(len >= 0 && len < (int64_t)GAE_CHUNK * (1LL << 30), TALOS_ERR_SHAPE, "bad rollout length");
  TALOS_REQUIRE(rew_var >= 0.f, TALOS_ERR_ARG, "reward variance must be non-negative");
  if (len == 0) return TALOS_OK;
  TALOS_REQUIRE(rewards && values && terminals && advantages && returns, TALOS_ERR_ARG, "null pointer");
  const int blocks = (int)ceil_div(len, GAE_CHUNK);
  char* ws = (char*)talos_workspace(ctx, (sizeof(Affine) + sizeof(float)) * (size_t)blocks + 16);
  Affine* maps = (Affine*)ws; float* carries = (float*)(maps + blocks);
  GaeArgs g{rewards, values, terminals, len, gamma, gamma * lambda, rew_mean, (float)(1.0 / (std::sqrt((double)rew_var) + 1e-8))};
  const int aligned = ((((uintptr_t)rewards | (uintptr_t)values | (uintptr_t)terminals | (uintptr_t)advantages | (uintptr_t)returns) & 15) == 0) ? 1 : 0;
  gae_scan_kernel<0><<<blocks, GAE_THREADS, 0, ctx->stream>>>(g, aligned, maps, nullptr, nullptr, nullptr);
  talos_launched(ctx, "gae_scan (fold)");
  gae_chain_kernel<<<1, CHAIN_THREADS, 0, ctx->stream>>>(maps, carries, blocks);
  talos_launched(ctx, "gae_chain");
  gae_scan_kernel<1><<<blocks, GAE_THREADS, 0, ctx->stream>>>(g, aligned, maps, carries, advantages, returns);
  talos_launched(ctx, "gae_scan (replay)");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_normalize_slice(talos_ctx* ctx, const float* x, int64_t n, float* y, float* stats) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "bad length");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(x && y, TALOS_ERR_ARG, "null pointer");
  const int blocks = (int)std::min<int64_t>(ceil_div(n, RED_THREADS * 8), 8 * ctx->sm_count);
  const int vec = ((((uintptr_t)x | (uintptr_t)y) & 15) == 0) ? 1 : 0;
  char* ws = (char*)talos_workspace(ctx, sizeof(double) * (size_t)blocks + 16);
  double* partials = (double*)ws;
  float* st = stats ? stats : (float*)(partials + blocks);
  moment_partial_kernel<0><<<blocks, RED_THREADS, 0, ctx->stream>>>(x, n, vec, st, partials);
  talos_launched(ctx, "moment_partial (sum)");
  moment_final_kernel<0><<<1, RED_THREADS, 0, ctx->stream>>>(partials, blocks, n, st);
  talos_launched(ctx, "moment_final (mean)");
  moment_partial_kernel<1><<<blocks, RED_THREADS, 0, ctx->stream>>>(x, n, vec, st, partials);
  talos_launched(ctx, "moment_partial (squared differences)");
  moment_final_kernel<1><<<1, RED_THREADS, 0, ctx->stream>>>(partials, blocks, n, st);
  talos_launched(ctx, "moment_final (std)");
  normalize_kernel<<<(unsigned)ceil_div(vec ? ceil_div(n, 4) : n, 256), 256, 0, ctx->stream>>>(x, n, vec, st, y);
  talos_launched(ctx, "normalize");
  TALOS_ENTRY_END
}
