// Batched rollout inference for the MLA policy: one new token for each of N independent simulations, each with its
// own KV ring and its own absolute position.  This is MultiHeadLatentAttention::forward_inference_cached
// (src/transformer.rs:688-841) followed by prune_kv_cache (:843-874) as the simulator drives them
// (src/sim.rs:171-175, :208, :578), batched over simulations: rotate the new rotary parts by the token position,
// assemble q = [q_c | rot(q_r)] and k = [k_c | rot(k_r)], append k and v_c to the cache, attend over the cached rows
// with scale 1/sqrt(dh+dr), no mask.  A ring of cap = context_len + 1 slots per (simulation, head) replaces
// "append, attend, then drop the oldest rows beyond context_len": the set of rows attended to is the same, and
// attention does not depend on their order because the rotation uses absolute positions.
#include "common.cuh"

namespace {

constexpr int DEC_WARPS = 8;

__device__ __forceinline__ float dec_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float dec_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per (simulation, head).  Layouts: q_c, k_c, v_c [N][H*dh]; q_r, k_r [N][H*dr] (Linear outputs, used as
// they come); k_cache [N][H][cap][dh+dr]; v_cache [N][H][cap][dh]; out [N][H*dh]; pos [N].
// VEC: dh+dr is a multiple of 4 and the cache base is 16-byte aligned, so key rows are read as float4.
template <bool VEC>
__global__ void __launch_bounds__(DEC_WARPS * 32)
mla_decode_kernel(const float* __restrict__ q_c, const float* __restrict__ q_r, const float* __restrict__ k_c,
                  const float* __restrict__ k_r, const float* __restrict__ v_c, const float* __restrict__ cos_t,
                  const float* __restrict__ sin_t, long long table_len, const int* __restrict__ pos, float* k_cache,
                  float* v_cache, float* __restrict__ out, long long items, int H, int dh, int dr, int cap, float scale) {
  extern __shared__ __align__(16) float dec_sm[];
  const int dk = dh + dr, dk_pad = (dk + 3) & ~3, cap_pad = (cap + 3) & ~3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = dec_sm + warp * (dk_pad + cap_pad);        // the query row (16-byte aligned), broadcast to every lane
  float* ps = qs + dk_pad;                               // scores, then unnormalised probabilities
  const long long item = (long long)blockIdx.x * DEC_WARPS + warp;   // = n * H + h
  if (item >= items) return;                             // whole warps leave; no block-wide barrier below
  const long long n = item / H;
  const int p = pos[n];
  const int slot = p % cap, live = min(p + 1, cap);
  float* const kbase = k_cache + item * cap * dk;
  float* const vbase = v_cache + item * cap * dh;
  float* const krow = kbase + (long long)slot * dk;
  float* const vrow = vbase + (long long)slot * dh;

  for (int c = lane; c < dh; c += 32) {
    qs[c] = q_c[item * dh + c];
    krow[c] = k_c[item * dh + c];
    vrow[c] = v_c[item * dh + c];
  }
  // Interleaved pairs (2i, 2i+1) rotated by the simulation's absolute position; a position whose table row lies
  // past the end of the table is left unrotated (src/transformer.rs:716-719).
  const long long toff = (long long)p * (dr / 2);
  const bool rotate = toff < table_len;
  for (int i = lane; i < dr / 2; i += 32) {
    const float c = rotate ? cos_t[toff + i] : 1.f, s = rotate ? sin_t[toff + i] : 0.f;
    const float q1 = q_r[item * dr + 2 * i], q2 = q_r[item * dr + 2 * i + 1];
    const float k1 = k_r[item * dr + 2 * i], k2 = k_r[item * dr + 2 * i + 1];
    qs[dh + 2 * i] = q1 * c - q2 * s; qs[dh + 2 * i + 1] = q1 * s + q2 * c;
    krow[dh + 2 * i] = k1 * c - k2 * s; krow[dh + 2 * i + 1] = k1 * s + k2 * c;
  }
  __syncwarp();                                          // the new key / value rows are read back by other lanes

  // scores: lane j owns ring slots j, j+32, ...
  float mx = -INFINITY;
  for (int j = lane; j < live; j += 32) {
    const float* kr = kbase + (long long)j * dk;
    float acc = 0.f;
    if (VEC) {
      for (int c = 0; c < dk; c += 4) {
        const float4 kv = *(const float4*)(kr + c), qv = *(const float4*)(qs + c);
        acc = fmaf(qv.x, kv.x, acc); acc = fmaf(qv.y, kv.y, acc); acc = fmaf(qv.z, kv.z, acc); acc = fmaf(qv.w, kv.w, acc);
      }
    } else {
      for (int c = 0; c < dk; ++c) acc = fmaf(qs[c], kr[c], acc);
    }
    acc *= scale; ps[j] = acc; mx = fmaxf(mx, acc);
  }
  mx = dec_warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < live; j += 32) { const float e = expf(ps[j] - mx); ps[j] = e; sum += e; }
  sum = dec_warp_sum(sum);
  const float inv = 1.f / sum;
  __syncwarp();

  // out[c] = sum_j p_j V[j][c]: lanes along the head dimension, rows streamed in ring order
  for (int c = lane; c < dh; c += 32) {
    float acc = 0.f;
    for (int j = 0; j < live; ++j) acc = fmaf(ps[j], vbase[(long long)j * dh + c], acc);
    out[item * dh + c] = acc * inv;
  }
}

__global__ void decode_advance_kernel(int* pos, const int* __restrict__ reset, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) pos[i] = (reset && reset[i]) ? 0 : pos[i] + 1;
}

}  // namespace

TALOS_API talos_status talos_mla_decode_step(talos_ctx* ctx, const float* q_c, const float* q_r, const float* k_c, const float* k_r,
                                             const float* v_c, const float* cos_t, const float* sin_t, int64_t table_len,
                                             const int32_t* pos, float* k_cache, float* v_cache, float* out, int64_t N, int64_t H,
                                             int64_t dh, int64_t dr, int64_t cap, float scale) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(N >= 0 && H >= 1 && H <= 1024 && dh >= 1 && dh <= 4096 && dr >= 0 && dr <= 4096 && (dr & 1) == 0 && cap >= 1 && cap <= 4096 && table_len >= 0,
                TALOS_ERR_SHAPE, "bad decode shape");
  if (N == 0) return TALOS_OK;
  TALOS_REQUIRE(q_c && k_c && v_c && pos && k_cache && v_cache && out, TALOS_ERR_ARG, "null pointer");
  TALOS_REQUIRE(dr == 0 || (q_r && k_r && cos_t && sin_t), TALOS_ERR_ARG, "rotary parts need q_r, k_r and the tables");
  const int64_t dk = dh + dr, items = N * H;
  const size_t shmem = sizeof(float) * DEC_WARPS * (size_t)(((dk + 3) & ~int64_t(3)) + ((cap + 3) & ~int64_t(3)));
  TALOS_REQUIRE(shmem <= 48 * 1024, TALOS_ERR_UNSUPPORTED, "decode step: head width + ring capacity too large");
  const unsigned grid = (unsigned)ceil_div(items, DEC_WARPS);
  const bool vec = (dk % 4 == 0) && (((uintptr_t)k_cache & 15) == 0);
  if (vec)
    mla_decode_kernel<true><<<grid, DEC_WARPS * 32, shmem, ctx->stream>>>(q_c, q_r, k_c, k_r, v_c, cos_t, sin_t, table_len, pos, k_cache, v_cache, out,
                                                                          items, (int)H, (int)dh, (int)dr, (int)cap, scale);
  else
    mla_decode_kernel<false><<<grid, DEC_WARPS * 32, shmem, ctx->stream>>>(q_c, q_r, k_c, k_r, v_c, cos_t, sin_t, table_len, pos, k_cache, v_cache, out,
                                                                           items, (int)H, (int)dh, (int)dr, (int)cap, scale);
  talos_launched(ctx, "mla_decode_step");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_decode_advance(talos_ctx* ctx, int32_t* pos, const int32_t* reset, int64_t N) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(N >= 0, TALOS_ERR_SHAPE, "bad count");
  if (N == 0) return TALOS_OK;
  TALOS_REQUIRE(pos, TALOS_ERR_ARG, "null pointer");
  decode_advance_kernel<<<(unsigned)ceil_div(N, 256), 256, 0, ctx->stream>>>(pos, reset, N);
  talos_launched(ctx, "decode_advance");
  TALOS_ENTRY_END
}
