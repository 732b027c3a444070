// Attention core for short sequences (S <= 128): one CTA per (batch, head) keeps Q, K^T, V and the
// S x S score tile in shared memory and runs scores -> scale -> (mask) -> softmax -> P.V without a
// round trip of the scores through HBM.  Q and K may each be given as two strided sources (a content
// part and a rotary part) so that MLA's concat + transpose + reshape chain
// (src/transformer.rs:508-533) never materialises.
#include "common.cuh"

// A [batch, head, seq, d] view of strided memory: element (b,h,s,c) = p[b*sb + h*sh + s*ss + c].
struct HeadView { const float* p; long long sb, sh, ss; int d; };
struct HeadViewOut { float* p; long long sb, sh, ss; int d; };

namespace {

template <int TS>
__global__ void __launch_bounds__(256)
attention_fwd_kernel(HeadView q1, HeadView q2, HeadView k1, HeadView k2, HeadView v, HeadViewOut out, float* probs,
                     int H, int S, float scale, int causal) {
  extern __shared__ float sm[];
  const int dqk = q1.d + q2.d, dv = v.d, SP = S + 1;
  float* Qs = sm;                       // [S][dqk]
  float* Kt = Qs + S * dqk;             // [dqk][SP]
  float* Sc = Kt + dqk * SP;            // [S][SP]
  float* Vs = Sc + S * SP;              // [S][dv]
  const int bh = blockIdx.x, b = bh / H, h = bh % H, tid = threadIdx.x;

  for (int e = tid; e < S * dqk; e += 256) {
    int s = e / dqk, c = e % dqk;
    float qv, kv;
    if (c < q1.d) { qv = q1.p[b * q1.sb + h * q1.sh + s * q1.ss + c]; kv = k1.p[b * k1.sb + h * k1.sh + s * k1.ss + c]; }
    else { int c2 = c - q1.d; qv = q2.p[b * q2.sb + h * q2.sh + s * q2.ss + c2]; kv = k2.p[b * k2.sb + h * k2.sh + s * k2.ss + c2]; }
    Qs[e] = qv; Kt[c * SP + s] = kv;
  }
  for (int e = tid; e < S * dv; e += 256) { int s = e / dv, c = e % dv; Vs[e] = v.p[b * v.sb + h * v.sh + s * v.ss + c]; }
  __syncthreads();

  const int tx = tid & 15, ty = tid >> 4;
  {
    float acc[TS][TS];
#pragma unroll
    for (int i = 0; i < TS; ++i)
#pragma unroll
      for (int j = 0; j < TS; ++j) acc[i][j] = 0.f;
    for (int c = 0; c < dqk; ++c) {
      float a[TS], bb[TS];
#pragma unroll
      for (int i = 0; i < TS; ++i) { int r = ty + 16 * i; a[i] = r < S ? Qs[r * dqk + c] : 0.f; }
#pragma unroll
      for (int j = 0; j < TS; ++j) { int cc = tx + 16 * j; bb[j] = cc < S ? Kt[c * SP + cc] : 0.f; }
#pragma unroll
      for (int i = 0; i < TS; ++i)
#pragma unroll
        for (int j = 0; j < TS; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TS; ++i)
#pragma unroll
      for (int j = 0; j < TS; ++j) { int r = ty + 16 * i, cc = tx + 16 * j; if (r < S && cc < S) Sc[r * SP + cc] = acc[i][j] * scale; }
  }
  __syncthreads();

  // softmax rows: warp w takes rows w, w+8, ...
  const int lane = tid & 31, w = tid >> 5;
  for (int r = w; r < S; r += 8) {
    const int lim = causal ? r + 1 : S;
    float mx = -INFINITY;
    for (int c = lane; c < lim; c += 32) mx = fmaxf(mx, Sc[r * SP + c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int c = lane; c < S; c += 32) { float e = c < lim ? expf(Sc[r * SP + c] - mx) : 0.f; Sc[r * SP + c] = e; sum += e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    for (int c = lane; c < S; c += 32) {
      float p = Sc[r * SP + c] * inv; Sc[r * SP + c] = p;
      if (probs) probs[((long long)bh * S + r) * S + c] = p;
    }
  }
  __syncthreads();

  // out = P.V : thread (ty,tx) owns rows ty+16i, columns tx+16j of [S][dv]
  constexpr int TV = 8;                                   // dv <= 128
  for (int j0 = 0; j0 < dv; j0 += 16 * TV) {
    float acc[TS][TV];
#pragma unroll
    for (int i = 0; i < TS; ++i)
#pragma unroll
      for (int j = 0; j < TV; ++j) acc[i][j] = 0.f;
    for (int c = 0; c < S; ++c) {
      float a[TS], bb[TV];
#pragma unroll
      for (int i = 0; i < TS; ++i) { int r = ty + 16 * i; a[i] = r < S ? Sc[r * SP + c] : 0.f; }
#pragma unroll
      for (int j = 0; j < TV; ++j) { int cc = j0 + tx + 16 * j; bb[j] = cc < dv ? Vs[c * dv + cc] : 0.f; }
#pragma unroll
      for (int i = 0; i < TS; ++i)
#pragma unroll
        for (int j = 0; j < TV; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TS; ++i)
#pragma unroll
      for (int j = 0; j < TV; ++j) {
        int r = ty + 16 * i, cc = j0 + tx + 16 * j;
        if (r < S && cc < dv) out.p[b * out.sb + h * out.sh + r * out.ss + cc] = acc[i][j];
      }
  }
}

}  // namespace

void talos_attention_launch(talos_ctx* ctx, HeadView q1, HeadView q2, HeadView k1, HeadView k2, HeadView v,
                            HeadViewOut out, float* probs, int64_t B, int H, int S, float scale, int causal) {
  const int dqk = q1.d + q2.d, dv = v.d;
  TALOS_REQUIRE(S >= 1 && S <= 128, TALOS_ERR_UNSUPPORTED, "attention core supports 1 <= S <= 128");
  TALOS_REQUIRE(dqk >= 1 && dqk <= 256 && dv >= 1 && dv <= 128, TALOS_ERR_UNSUPPORTED, "attention head dims out of range");
  size_t shmem = sizeof(float) * ((size_t)S * dqk + (size_t)dqk * (S + 1) + (size_t)S * (S + 1) + (size_t)S * dv);
  TALOS_REQUIRE(shmem <= 227 * 1024, TALOS_ERR_UNSUPPORTED, "attention tile does not fit in shared memory");
  const int ts = (S + 15) / 16;
  auto launch = [&](auto kern) {
    TALOS_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shmem));
    kern<<<(unsigned)(B * H), 256, shmem, ctx->stream>>>(q1, q2, k1, k2, v, out, probs, H, S, scale, causal);
  };
  if (ts <= 1) launch(attention_fwd_kernel<1>);
  else if (ts <= 2) launch(attention_fwd_kernel<2>);
  else if (ts <= 4) launch(attention_fwd_kernel<4>);
  else launch(attention_fwd_kernel<8>);
  talos_launched(ctx, "attention_fwd");
}

// Tensor-core route of the forward pass (TF32 / 3xTF32 modes): scores = Q.K^T as one batched tensor-core GEMM written
// to `sc` (the caller's probs buffer, or scratch), softmax in place, out = P.V as a second batched GEMM.  The scores
// make one round trip through HBM (~4 S^2 x 4 bytes per head), which at S = 128 still costs a tenth of the fused
// CUDA-core kernel's arithmetic time.  Returns false when the tensor-core GEMM does not take the shape.
bool talos_attention_tc_fused(talos_ctx* ctx, const float* q, const float* k, const float* v, float* out, float* probs, int64_t BH,
                              int64_t S, int64_t dqk, int64_t dv, float scale, int causal);

static bool attention_fwd_tc(talos_ctx* ctx, const float* q, const float* k, const float* v, float* out, float* probs,
                             int64_t BH, int64_t S, int64_t dqk, int64_t dv, float scale, int causal, int mode) {
  // fast mode, S <= 128: one fused kernel with the scores in tensor memory (attention_tc.cu)
  if (mode == TALOS_MODE_TF32 && talos_attention_tc_fused(ctx, q, k, v, out, probs, BH, S, dqk, dv, scale, causal)) return true;
  if (S > 1024) return false;                                       // row softmax limit
  float* sc = probs ? probs : (float*)talos_workspace2(ctx, sizeof(float) * (size_t)(BH * S * S));
  const EpiArgs none = talos_epi_args(nullptr);
  if (!talos_gemm_tc_launch_batched(ctx, TALOS_OP_N, TALOS_OP_T, S, S, dqk, q, dqk, S * dqk, k, dqk, S * dqk, sc, S, S * S, BH, mode, none))
    return false;
  talos_status st = talos_softmax_fwd(ctx, sc, sc, BH * S, S, scale, causal ? S : 0);
  if (st != TALOS_OK) throw talos_error(st, talos_last_error_string());
  st = talos_gemm_batched(ctx, TALOS_OP_N, TALOS_OP_N, S, dv, S, sc, S, S * S, v, dv, S * dv, out, dv, S * dv, BH, 0, mode);
  if (st != TALOS_OK) throw talos_error(st, talos_last_error_string());
  return true;
}

TALOS_API talos_status talos_attention_fwd(talos_ctx* ctx, const float* q, const float* k, const float* v, float* out,
                                           float* probs, int64_t BH, int64_t S, int64_t dqk, int64_t dv, float scale,
                                           int32_t causal, int32_t mode) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(BH >= 0 && S >= 0 && dqk >= 1 && dv >= 1, TALOS_ERR_SHAPE, "bad attention shape");
  TALOS_REQUIRE(mode >= TALOS_MODE_FP32 && mode <= TALOS_MODE_TF32, TALOS_ERR_ARG, "bad arithmetic mode");
  if (BH == 0 || S == 0) return TALOS_OK;
  TALOS_REQUIRE(q && k && v && out, TALOS_ERR_ARG, "null pointer");
  if (mode != TALOS_MODE_FP32 && attention_fwd_tc(ctx, q, k, v, out, probs, BH, S, dqk, dv, scale, causal ? 1 : 0, mode)) return TALOS_OK;
  HeadView none{nullptr, 0, 0, 0, 0};
  talos_attention_launch(ctx, HeadView{q, S * dqk, 0, dqk, (int)dqk}, none, HeadView{k, S * dqk, 0, dqk, (int)dqk}, none,
                         HeadView{v, S * dv, 0, dv, (int)dv}, HeadViewOut{out, S * dv, 0, dv, (int)dv}, probs, BH, 1, (int)S,
                         scale, causal ? 1 : 0);
  TALOS_ENTRY_END
}

// Backward from the saved probabilities, as the product of the reference's four closures
// (src/transformer.rs:1010-1046, :1098-1117, :1063-1068, :920-955):
//   dV = P^T.dO ; dP = dO.V^T ; dS = scale * P * (dP - rowsum(dP*P)) ; dQ = dS.K ; dK = dS^T.Q
// The four products are batched GEMMs in the requested arithmetic mode (tensor cores for TF32 / 3xTF32).
TALOS_API talos_status talos_attention_bwd(talos_ctx* ctx, const float* q, const float* k, const float* v,
                                           const float* probs, const float* dout, float* dq, float* dk, float* dv,
                                           int64_t BH, int64_t S, int64_t dqk, int64_t dvd, float scale, int32_t mode) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(BH >= 0 && S >= 0 && dqk >= 1 && dvd >= 1 && S <= 1024, TALOS_ERR_SHAPE, "bad attention shape");
  TALOS_REQUIRE(mode >= TALOS_MODE_FP32 && mode <= TALOS_MODE_TF32, TALOS_ERR_ARG, "bad arithmetic mode");
  if (BH == 0 || S == 0) return TALOS_OK;
  TALOS_REQUIRE(q && k && v && probs && dout && dq && dk && dv, TALOS_ERR_ARG, "null pointer");
  float* dS = (float*)talos_workspace2(ctx, sizeof(float) * (size_t)(BH * S * S));
  talos_status st;
  st = talos_gemm_batched(ctx, TALOS_OP_T, TALOS_OP_N, S, dvd, S, probs, S, S * S, dout, dvd, S * dvd, dv, dvd, S * dvd, BH, 0, mode);
  if (st) return st;
  st = talos_gemm_batched(ctx, TALOS_OP_N, TALOS_OP_T, S, S, dvd, dout, dvd, S * dvd, v, dvd, S * dvd, dS, S, S * S, BH, 0, mode);
  if (st) return st;
  st = talos_softmax_bwd(ctx, probs, dS, dS, BH * S, S, scale, 0);
  if (st) return st;
  st = talos_gemm_batched(ctx, TALOS_OP_N, TALOS_OP_N, S, dqk, S, dS, S, S * S, k, dqk, S * dqk, dq, dqk, S * dqk, BH, 0, mode);
  if (st) return st;
  st = talos_gemm_batched(ctx, TALOS_OP_T, TALOS_OP_N, S, dqk, S, dS, S, S * S, q, dqk, S * dqk, dk, dqk, S * dqk, BH, 0, mode);
  if (st) return st;
  TALOS_ENTRY_END
}
