// PPO clipped-surrogate loss (forward + gradient in one pass) and the Adam optimizer step.
#include "common.cuh"

namespace {

constexpr int MAX_ACTIONS = 64;

// One thread per transition.  Restates the per-sample graph of PPO::update (src/ppo.rs:702-755):
// max-subtracted log-softmax, ratio = exp(logp[a] - old), kl = (ratio-1) - log_ratio, surr1 is the
// policy term iff surr1 < surr2, clip passes gradient on the closed interval, v_loss = (v-R)^2,
// H = -sum p logp; loss = -policy + c_v v_loss - c_h H.  Gradients are divided by `denom`.
template <int A>
__global__ void __launch_bounds__(128)
ppo_loss_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ values, long long vs,
                const int* __restrict__ actions, const float* __restrict__ old_logp, const float* __restrict__ adv,
                const float* __restrict__ ret, long long n, int n_actions, float clip, float c_v, float c_h, float inv_denom,
                float* __restrict__ dlogits, long long ld_out, float* __restrict__ dvalues, long long dvs,
                float* __restrict__ partial, int vec, int32_t* __restrict__ status, float* __restrict__ colsum_part, int cs_width) {
  __shared__ float sh_loss[128], sh_kl[128];
  __shared__ float sh_cs[4][MAX_ACTIONS + 1];
  const bool want_cs = colsum_part != nullptr;                 // block-uniform
  const int na_cs = A > 0 ? A : n_actions;
  float dv_out = 0.f;
  float l_keep[A > 0 ? A : 1];                                 // this row's dlogits, for the column sums (specialised widths only)
#pragma unroll
  for (int a = 0; a < (A > 0 ? A : 1); ++a) l_keep[a] = 0.f;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float loss = 0.f, kl = 0.f;
  if (i < n) {
    const int na = A > 0 ? A : n_actions;
    float l[A > 0 ? A : MAX_ACTIONS];
    float mx = -INFINITY;
    // each thread owns one row: 128-bit accesses when the row is a whole number of aligned float4 (the host checks)
    constexpr bool VEC = (A > 0) && (A % 4 == 0);
    if (VEC && vec) {
#pragma unroll
      for (int a = 0; a < na; a += 4) {
        const float4 q = *(const float4*)(logits + i * ld + a);
        l[a] = q.x; l[a + 1] = q.y; l[a + 2] = q.z; l[a + 3] = q.w;
      }
#pragma unroll
      for (int a = 0; a < na; ++a) mx = fmaxf(mx, l[a]);
    } else {
#pragma unroll
      for (int a = 0; a < na; ++a) { l[a] = logits[i * ld + a]; mx = fmaxf(mx, l[a]); }
    }
    float se = 0.f;
#pragma unroll
    for (int a = 0; a < na; ++a) se += expf(l[a] - mx);
    const float lse = logf(se) + mx;
    const int act = actions[i];
    // An action outside [0, na) would match no logit below and yield a plausible-looking loss: report it instead
    // (the sample then contributes its entropy and value terms only).
    if (act < 0 || act >= na) atomicExch(status, TALOS_DEV_BAD_INDEX);
    const float advantage = adv[i];
    float ent = 0.f, lp_a = 0.f, sum_d = 0.f;
#pragma unroll
    for (int a = 0; a < na; ++a) {
      float lp = l[a] - lse, p = expf(lp);
      ent -= p * lp;
      if (a == act) lp_a = lp;
      l[a] = lp;
    }
    const float log_ratio = lp_a - old_logp[i], ratio = expf(log_ratio);
    kl = (ratio - 1.f) - log_ratio;
    const float lo = 1.f - clip, hi = 1.f + clip;
    const float surr1 = ratio * advantage, surr2 = fminf(fmaxf(ratio, lo), hi) * advantage;
    const bool use1 = surr1 < surr2;
    const float policy = use1 ? surr1 : surr2;
    const float d_ratio = use1 ? advantage : ((ratio >= lo && ratio <= hi) ? advantage : 0.f);
    const float v = values[i * vs], dvl = v - ret[i];
    loss = -policy + c_v * dvl * dvl - c_h * ent;
    const float d_lp_a = -(d_ratio * ratio);
    // d(loss)/d logp_j = c_h p_j (logp_j + 1) [+ d_lp_a at j = a]; logp = logits - lse
#pragma unroll
    for (int a = 0; a < na; ++a) {
      float lp = l[a], p = expf(lp);
      float d = c_h * p * (lp + 1.f) + (a == act ? d_lp_a : 0.f);
      sum_d += d; l[a] = d;
    }
    // p_j again from logp_j = log p_j: kept as p in a second pass to spare registers
    if (VEC && vec) {
#pragma unroll
      for (int a = 0; a < na; a += 4) {
        const float4 q = *(const float4*)(logits + i * ld + a);
        float4 o;
        o.x = (l[a] - expf(q.x - lse) * sum_d) * inv_denom; o.y = (l[a + 1] - expf(q.y - lse) * sum_d) * inv_denom;
        o.z = (l[a + 2] - expf(q.z - lse) * sum_d) * inv_denom; o.w = (l[a + 3] - expf(q.w - lse) * sum_d) * inv_denom;
        *(float4*)(dlogits + i * ld_out + a) = o;
        if (A > 0) { l_keep[a] = o.x; l_keep[a + 1] = o.y; l_keep[a + 2] = o.z; l_keep[a + 3] = o.w; }
      }
    } else {
#pragma unroll
      for (int a = 0; a < na; ++a) {
        float lp_p = expf(logits[i * ld + a] - lse); const float o = (l[a] - lp_p * sum_d) * inv_denom;
        dlogits[i * ld_out + a] = o;
        if (A > 0) l_keep[a] = o;
      }
    }
    dv_out = c_v * 2.f * dvl * inv_denom;
    dvalues[i * dvs] = dv_out;
  }
  if (A > 0 && want_cs) {
    // Column sums of this block's rows of [dlogits | dvalue | zero padding] (the fused heads' bias gradient): warp
    // shuffles per column, then the four warps' sums in warp order.
    const int w = threadIdx.x >> 5, ln = threadIdx.x & 31;
#pragma unroll
    for (int a = 0; a <= A; ++a) {
      float v = a < A ? l_keep[a < A ? a : 0] : dv_out;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (ln == 0) sh_cs[w][a] = v;
    }
    __syncthreads();
    if ((int)threadIdx.x < cs_width) {
      const int a = threadIdx.x;
      colsum_part[(size_t)blockIdx.x * cs_width + a] = a <= na_cs ? ((sh_cs[0][a] + sh_cs[1][a]) + (sh_cs[2][a] + sh_cs[3][a])) : 0.f;
    }
  }
  sh_loss[threadIdx.x] = loss; sh_kl[threadIdx.x] = kl; __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (threadIdx.x < o) { sh_loss[threadIdx.x] += sh_loss[threadIdx.x + o]; sh_kl[threadIdx.x] += sh_kl[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { partial[2 * blockIdx.x] = sh_loss[0]; partial[2 * blockIdx.x + 1] = sh_kl[0]; }
}

// Sums the per-block (loss, kl) partials in block order and adds {loss, kl, n} to stats.
__global__ void ppo_stats_kernel(const float* __restrict__ partial, int nblocks, float n, float* stats) {
  __shared__ float sl[256], sk[256];
  float a = 0.f, b = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += 256) { a += partial[2 * i]; b += partial[2 * i + 1]; }
  sl[threadIdx.x] = a; sk[threadIdx.x] = b; __syncthreads();
  for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) { sl[threadIdx.x] += sl[threadIdx.x + o]; sk[threadIdx.x] += sk[threadIdx.x + o]; } __syncthreads(); }
  if (threadIdx.x == 0) { stats[0] += sl[0]; stats[1] += sk[0]; stats[2] += n; }
}

__global__ void sumsq_stage1_kernel(const float* __restrict__ g, long long n, float scale, float* __restrict__ partial) {
  __shared__ float sh[256];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) { float v = g[i] * scale; s += v * v; }
  sh[threadIdx.x] = s; __syncthreads();
  for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o]; __syncthreads(); }
  if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}

// Adam::step (src/ppo.rs:519-533).  norm_partial != null: DQN's global-norm clip (src/dqn.rs:209-222);
// every thread re-sums the (few) block partials in the same order, so the result is deterministic.
__global__ void adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                            long long n, float lr, float b1, float b2, float eps, float inv_bc1, float inv_bc2,
                            float grad_scale, const float* __restrict__ norm_partial, int nparts, float clip_norm,
                            const float* __restrict__ count_ptr, float* __restrict__ stats_out) {
  float coef = grad_scale;
  if (count_ptr) {                       // gradients hold sums over `count` samples (the tail of the flat buffer)
    coef = grad_scale / fmaxf(count_ptr[0], 1.f);
    if (stats_out && blockIdx.x == 0 && threadIdx.x < 4) stats_out[threadIdx.x] = count_ptr[(int)threadIdx.x - 2];
  }
  if (norm_partial) {
    float tot = 0.f;
    for (int i = 0; i < nparts; ++i) tot += norm_partial[i];
    tot = sqrtf(tot);
    if (tot > clip_norm) coef *= clip_norm / tot;
  }
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float gi = g[i] * coef;
  float mi = b1 * m[i] + (1.f - b1) * gi;
  float vi = b2 * v[i] + (1.f - b2) * gi * gi;
  m[i] = mi; v[i] = vi;
  p[i] -= lr * (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
}

}  // namespace

// The loss kernel alone: per-block {loss, kl} sums into partial[blocks][2] (blocks = ceil(n / 128), returned) and,
// when colsum_part is given (widths the kernel is specialised for, the value gradient in column n_actions of the
// same rows), per-block column sums of [dlogits | dvalue | 0...] into colsum_part[blocks][cs_width].
int talos_ppo_loss_launch(talos_ctx* ctx, const float* logits, int64_t ld_logits, const float* values, int64_t value_stride, const int32_t* actions,
                          const float* old_logp, const float* adv, const float* ret, int64_t n, int32_t n_actions, float clip, float c_value,
                          float c_entropy, float denom, float* dlogits, int64_t ld_out, float* dvalues, int64_t dvalue_stride, float* partial,
                          float* colsum_part, int cs_width) {
  const int blocks = (int)ceil_div(n, 128);
#define TALOS_PPO_LAUNCH(A) ppo_loss_kernel<A><<<blocks, 128, 0, ctx->stream>>>(logits, ld_logits, values, value_stride, actions, old_logp, adv, ret, n, n_actions, clip, c_value, c_entropy, 1.f / denom, dlogits, ld_out, dvalues, dvalue_stride, partial, vec, ctx->dev_status, colsum_part, cs_width)
  const int vec = (((uintptr_t)logits | (uintptr_t)dlogits) & 15) == 0 && ld_logits % 4 == 0 && ld_out % 4 == 0;
  if (n_actions == 16) TALOS_PPO_LAUNCH(16); else if (n_actions == 5) TALOS_PPO_LAUNCH(5); else TALOS_PPO_LAUNCH(0);
#undef TALOS_PPO_LAUNCH
  talos_launched(ctx, "ppo_loss");
  return blocks;
}
bool talos_ppo_loss_colsum_supported(int32_t n_actions, int cs_width) { return (n_actions == 16 || n_actions == 5) && cs_width > n_actions && cs_width <= 128; }

TALOS_API talos_status talos_ppo_loss_fwd_bwd(talos_ctx* ctx, const float* logits, int64_t ld_logits, const float* values,
                                              int64_t value_stride, const int32_t* actions, const float* old_logp,
                                              const float* adv, const float* ret, int64_t n, int32_t n_actions, float clip,
                                              float c_value, float c_entropy, float denom, float* dlogits, int64_t ld_out,
                                              float* dvalues, int64_t dvalue_stride, float* stats) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0 && n_actions >= 1 && n_actions <= MAX_ACTIONS, TALOS_ERR_SHAPE, "1..64 actions supported");
  TALOS_REQUIRE(ld_logits >= n_actions && ld_out >= n_actions && denom > 0.f, TALOS_ERR_SHAPE, "bad leading dimension or denominator");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(logits && values && actions && old_logp && adv && ret && dlogits && dvalues && stats, TALOS_ERR_ARG, "null pointer");
  int blocks = (int)ceil_div(n, 128);
  float* partial = (float*)talos_workspace(ctx, sizeof(float) * 2 * (size_t)blocks);
  talos_ppo_loss_launch(ctx, logits, ld_logits, values, value_stride, actions, old_logp, adv, ret, n, n_actions, clip, c_value, c_entropy, denom, dlogits,
                        ld_out, dvalues, dvalue_stride, partial, nullptr, 0);
  ppo_stats_kernel<<<1, 256, 0, ctx->stream>>>(partial, blocks, (float)n, stats);
  talos_launched(ctx, "ppo_stats");
  TALOS_ENTRY_END
}

void talos_adam_launch(talos_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n, int64_t t, float lr,
                       float beta1, float beta2, float eps, float grad_scale, const float* count_ptr, float clip_norm,
                       float* stats_out) {
  const double bc1 = 1.0 - pow((double)beta1, (double)t), bc2 = 1.0 - pow((double)beta2, (double)t);
  float* norm_partial = nullptr; int nparts = 0;
  if (clip_norm > 0.f) {
    nparts = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n, 4096), 64));
    norm_partial = (float*)talos_workspace(ctx, sizeof(float) * nparts);
    sumsq_stage1_kernel<<<nparts, 256, 0, ctx->stream>>>(grads, n, grad_scale, norm_partial);
    talos_launched(ctx, "adam_sumsq");
  }
  adam_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(params, grads, m, v, n, lr, beta1, beta2, eps, (float)(1.0 / bc1),
                                                                  (float)(1.0 / bc2), grad_scale, norm_partial, nparts, clip_norm,
                                                                  count_ptr, stats_out);
  talos_launched(ctx, "adam");
}

TALOS_API talos_status talos_adam_step_global_clip(talos_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n,
                                                   int64_t t, float lr, float beta1, float beta2, float eps, float grad_scale,
                                                   const float* sumsq_dev, float clip_norm) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0 && t >= 1 && clip_norm > 0.f, TALOS_ERR_ARG, "Adam step number must be >= 1 and the clip norm positive");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(params && grads && m && v && sumsq_dev, TALOS_ERR_ARG, "null pointer");
  const double bc1 = 1.0 - pow((double)beta1, (double)t), bc2 = 1.0 - pow((double)beta2, (double)t);
  adam_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(params, grads, m, v, n, lr, beta1, beta2, eps, (float)(1.0 / bc1), (float)(1.0 / bc2),
                                                                  grad_scale, sumsq_dev, 1, clip_norm, nullptr, nullptr);
  talos_launched(ctx, "adam_global_clip");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_adam_step(talos_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n,
                                       int64_t t, float lr, float beta1, float beta2, float eps, float grad_scale,
                                       float clip_norm) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0 && t >= 1, TALOS_ERR_ARG, "Adam step number must be >= 1");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(params && grads && m && v, TALOS_ERR_ARG, "null pointer");
  talos_adam_launch(ctx, params, grads, m, v, n, t, lr, beta1, beta2, eps, grad_scale, nullptr, clip_norm, nullptr);
  TALOS_ENTRY_END
}
