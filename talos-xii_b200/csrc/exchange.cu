// Gradient exchange fused with the optimizer step, over NVLink peer memory.
//
// The data-parallel PPO update needs, once per optimizer step, the sum over ranks of ~90 000 gradient floats and then
// the same Adam step on every rank (src/ppo.rs:519-533 applied to the summed gradient).  That is a latency-sized
// exchange: through NCCL it costs a collective launch plus two more kernels (Adam, weight preparation) and 15-40 us
// that nothing overlaps.  Here ONE kernel does all of it: every rank publishes its local sums in an exchange slot that
// its peers have mapped (CUDA IPC), raises a sequence flag in every peer's area, waits until all flags have arrived,
// then every thread loads its four gradients from every rank's slot with plain peer loads, adds them IN RANK ORDER (so
// every rank computes bit-identical sums and its weights never drift apart), applies Adam and writes the TF32-prepared
// copies of the new weights for the next step's products.
//
// Every wait is bounded: a rank whose peers never publish gives up after `spins` polls, raises the context's error word
// (reported as TALOS_ERR_TIMEOUT by the next blocking call) and leaves the parameters untouched.  No multicast, no
// multimem: plain loads and stores on peer addresses.
#include "comm.cuh"

namespace {

__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer4(const float* p) {       // peer memory: volatile-style load, never from a stale line
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float round_tf32(float a) { return __uint_as_float((__float_as_uint(a) + 0x1000u) & 0xFFFFE000u); }

constexpr unsigned XCHG_DEFAULT_SPINS = 1u << 22;

__global__ void __launch_bounds__(256)
xchg_adam_kernel(XchgAdamArgs a) {
  __shared__ int sh_ok;
  __shared__ float sh_count;
  if (threadIdx.x == 0) {
    // Publish: the local sums were written by earlier kernels on this stream, so they are complete; ONE system fence
    // orders them before the flags for observers on other GPUs, and the flag stores themselves go out back to back.
    if (blockIdx.x == 0 && !a.skip_signal) {
      __threadfence_system();
      for (int r = 0; r < a.world; ++r) st_relaxed_sys(a.peer_flags[r] + a.rank, a.seq);
    }
    // Wait for every rank's publication of this sequence number in OUR area (bounded).
    int ok = 1;
    const unsigned long long* mine = a.peer_flags[a.rank];
    for (int r = 0; r < a.world && ok; ++r) {
      if (r == a.rank) continue;                         // our own sums are complete by stream order
      unsigned i = 0;
      while (ld_acquire_sys(mine + r) < a.seq) {
        if (++i >= a.spins) { ok = 0; break; }
        if (i > 1024) __nanosleep(200);
      }
    }
    if (!ok) atomicExch(a.status, TALOS_DEV_TIMEOUT_BASE + 1900 + a.rank);
    sh_ok = ok;
  }
  __syncthreads();
  if (!sh_ok) return;                                   // nothing is updated on a rank that gave up
  const long long i4 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long n4 = a.n >> 2;
  const bool active = i4 <= n4;
  // Every peer load of this thread is issued before the first one is used: a remote load is a round trip over NVLink,
  // and with eight ranks eight dependent round trips were most of the exchange's cost.
  float4 x[TALOS_MAX_RANKS], t[TALOS_MAX_RANKS];
#pragma unroll
  for (int r = 0; r < TALOS_MAX_RANKS; ++r) if (r < a.world && active) x[r] = ld_peer4(a.slot[r] + 4 * i4);
  if (threadIdx.x == 0) {                                // tail = {sum loss, sum kl, count, -}
#pragma unroll
    for (int r = 0; r < TALOS_MAX_RANKS; ++r) if (r < a.world) t[r] = ld_peer4(a.slot[r] + a.n);
    float cnt = 0.f;
#pragma unroll
    for (int r = 0; r < TALOS_MAX_RANKS; ++r) if (r < a.world) cnt += t[r].z;
    sh_count = cnt;
  }
  __syncthreads();
  if (!active) return;
  const float coef = 1.f / fmaxf(sh_count, 1.f);
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < TALOS_MAX_RANKS; ++r)              // rank order: the same sum on every rank
    if (r < a.world) { g.x += x[r].x; g.y += x[r].y; g.z += x[r].z; g.w += x[r].w; }
  if (a.grads_out) ((float4*)a.grads_out)[i4] = g;     // the reduced sums (and, in the last group, the reduced tail)
  if (i4 == n4) { if (a.stats_out) ((float4*)a.stats_out)[0] = g; return; }
  float4 p = ((float4*)a.params)[i4], m = ((float4*)a.m)[i4], v = ((float4*)a.v)[i4];
#define TALOS_ADAM_LANE(c)                                                              \
  { const float gi = g.c * coef; m.c = a.b1 * m.c + (1.f - a.b1) * gi; v.c = a.b2 * v.c + (1.f - a.b2) * gi * gi; \
    p.c -= a.lr * (m.c * a.inv_bc1) / (sqrtf(v.c * a.inv_bc2) + a.eps); }
  TALOS_ADAM_LANE(x) TALOS_ADAM_LANE(y) TALOS_ADAM_LANE(z) TALOS_ADAM_LANE(w)
#undef TALOS_ADAM_LANE
  ((float4*)a.params)[i4] = p; ((float4*)a.m)[i4] = m; ((float4*)a.v)[i4] = v;
  if (a.w_hi) {
    const float4 h = make_float4(round_tf32(p.x), round_tf32(p.y), round_tf32(p.z), round_tf32(p.w));
    ((float4*)a.w_hi)[i4] = h;
    if (a.w_lo) ((float4*)a.w_lo)[i4] = make_float4(round_tf32(p.x - h.x), round_tf32(p.y - h.y), round_tf32(p.z - h.z), round_tf32(p.w - h.w));
  }
}

}  // namespace

void talos_xchg_adam_launch(talos_ctx* ctx, const XchgAdamArgs& a_in) {
  XchgAdamArgs a = a_in;
  if (a.spins == 0) a.spins = XCHG_DEFAULT_SPINS;
  const long long groups = (a.n >> 2) + 1;             // + the tail group
  xchg_adam_kernel<<<(unsigned)ceil_div(groups, 256), 256, 0, ctx->stream>>>(a);
  talos_launched(ctx, "xchg_adam");
}
