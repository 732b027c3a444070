// The elementwise pieces of the dueling double-DQN train step (src/dqn.rs:68-107, :129-150, :482-584) as fused
// kernels; the Linear layers around them are GEMMs.  Batches here are small (64 in the crate), so everything is one
// thread per row or per element and the cost is launch latency.
#include "common.cuh"

namespace {

// q[b][a] = v[b] + adv[b][a] - mean_a(adv[b][:])                     (src/dqn.rs:76-93: the three matmuls with ones)
__global__ void dueling_fwd_kernel(const float* __restrict__ v, const float* __restrict__ adv, float* __restrict__ q, long long B, int A) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float s = 0.f;
  for (int a = 0; a < A; ++a) s += adv[b * A + a];
  const float base = v[b] - s / (float)A;
  for (int a = 0; a < A; ++a) q[b * A + a] = base + adv[b * A + a];
}
// dv[b] (+)= sum_a dq[b][a];  dadv[b][a] (+)= dq[b][a] - mean_a(dq[b][:])
__global__ void dueling_bwd_kernel(const float* __restrict__ dq, float* __restrict__ dv, float* __restrict__ dadv, long long B, int A, int acc) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float s = 0.f;
  for (int a = 0; a < A; ++a) s += dq[b * A + a];
  if (dv) dv[b] = acc ? dv[b] + s : s;
  if (dadv) {
    const float m = s / (float)A;
    for (int a = 0; a < A; ++a) { const float g = dq[b * A + a] - m; dadv[b * A + a] = acc ? dadv[b * A + a] + g : g; }
  }
}
// Double DQN (src/dqn.rs:524-556): the online network picks the action (first maximum wins, strict >), the target
// network values it: target[b] = r[b] + gamma * Qt[b][argmax_a Qe[b][a]] * (1 - done[b]).
__global__ void dqn_target_kernel(const float* __restrict__ q_eval, const float* __restrict__ q_target, const float* __restrict__ rewards,
                                  const float* __restrict__ dones, float gamma, float* __restrict__ target, long long B, int A) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int best = 0; float mx = -INFINITY;
  for (int a = 0; a < A; ++a) { const float x = q_eval[b * A + a]; if (x > mx) { mx = x; best = a; } }
  target[b] = rewards[b] + gamma * q_target[b * A + best] * (1.f - dones[b]);
}
// q_sel[b] = q[b][action[b]] (the mask-multiply + matmul with ones of src/dqn.rs:516-520); loss = mean_b (q_sel - t)^2
// (mse_loss, src/autograd.rs:1599-1603); dq[b][a] = 2 (q_sel - t) / B at the taken action, 0 elsewhere.
// One block; partial sums are combined in thread order, so the loss is reproducible.
__global__ void __launch_bounds__(256)
dqn_loss_kernel(const float* __restrict__ q, const int32_t* __restrict__ actions, const float* __restrict__ target, float* __restrict__ loss,
                float* __restrict__ dq, long long B, int A, int32_t* __restrict__ status) {
  __shared__ double sh[256];
  double acc = 0.0;
  for (long long b = threadIdx.x; b < B; b += 256) {
    const int act = actions[b];
    if (act < 0 || act >= A) {                         // a stale action buffer must not become a wild read: skip the sample, report it
      atomicExch(status, TALOS_DEV_BAD_INDEX);
      if (dq) for (int a = 0; a < A; ++a) dq[b * A + a] = 0.f;
      continue;
    }
    const float d = q[b * A + act] - target[b];
    acc += (double)d * d;
    if (dq) for (int a = 0; a < A; ++a) dq[b * A + a] = (a == act) ? 2.f * d / (float)B : 0.f;
  }
  sh[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x == 0) { double s = 0.0; for (int i = 0; i < 256; ++i) s += sh[i]; loss[0] = (float)(s / (double)B); }
}
// target <- target * (1 - tau) + source * tau                           (src/dqn.rs:129-150)
__global__ void soft_update_kernel(float* __restrict__ t, const float* __restrict__ s, float tau, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) t[i] = t[i] * (1.f - tau) + s[i] * tau;
}

}  // namespace

TALOS_API talos_status talos_dueling_combine_fwd(talos_ctx* ctx, const float* v, const float* adv, float* q, int64_t B, int64_t A) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(B >= 0 && A >= 1 && A <= 4096, TALOS_ERR_SHAPE, "bad dueling shape");
  if (B == 0) return TALOS_OK;
  TALOS_REQUIRE(v && adv && q, TALOS_ERR_ARG, "null pointer");
  dueling_fwd_kernel<<<(unsigned)ceil_div(B, 128), 128, 0, ctx->stream>>>(v, adv, q, B, (int)A);
  talos_launched(ctx, "dueling_fwd");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_dueling_combine_bwd(talos_ctx* ctx, const float* dq, float* dv, float* dadv, int64_t B, int64_t A, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(B >= 0 && A >= 1 && A <= 4096, TALOS_ERR_SHAPE, "bad dueling shape");
  if (B == 0) return TALOS_OK;
  TALOS_REQUIRE(dq && (dv || dadv), TALOS_ERR_ARG, "null pointer");
  dueling_bwd_kernel<<<(unsigned)ceil_div(B, 128), 128, 0, ctx->stream>>>(dq, dv, dadv, B, (int)A, accumulate ? 1 : 0);
  talos_launched(ctx, "dueling_bwd");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_dqn_target(talos_ctx* ctx, const float* q_next_eval, const float* q_next_target, const float* rewards,
                                        const float* dones, float gamma, float* target, int64_t B, int64_t A) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(B >= 0 && A >= 1 && A <= 4096, TALOS_ERR_SHAPE, "bad DQN target shape");
  if (B == 0) return TALOS_OK;
  TALOS_REQUIRE(q_next_eval && q_next_target && rewards && dones && target, TALOS_ERR_ARG, "null pointer");
  dqn_target_kernel<<<(unsigned)ceil_div(B, 128), 128, 0, ctx->stream>>>(q_next_eval, q_next_target, rewards, dones, gamma, target, B, (int)A);
  talos_launched(ctx, "dqn_target");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_dqn_loss_fwd_bwd(talos_ctx* ctx, const float* q, const int32_t* actions, const float* target, float* loss,
                                              float* dq, int64_t B, int64_t A) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(B >= 1 && A >= 1 && A <= 4096, TALOS_ERR_SHAPE, "bad DQN loss shape");
  TALOS_REQUIRE(q && actions && target && loss, TALOS_ERR_ARG, "null pointer");
  dqn_loss_kernel<<<1, 256, 0, ctx->stream>>>(q, actions, target, loss, dq, B, (int)A, ctx->dev_status);
  talos_launched(ctx, "dqn_loss");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_soft_update(talos_ctx* ctx, float* target_params, const float* source_params, float tau, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0, TALOS_ERR_SHAPE, "bad length");
  if (n == 0) return TALOS_OK;
  TALOS_REQUIRE(target_params && source_params, TALOS_ERR_ARG, "null pointer");
  soft_update_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(target_params, source_params, tau, n);
  talos_launched(ctx, "soft_update");
  TALOS_ENTRY_END
}
