// Fused attention forward on the tensor cores (fast TF32 mode): scores -> scale -> softmax -> . V for one (batch, head)
// per tile, with the S x S scores living in tensor memory and never touching HBM.  Replaces, for S <= 128, the two
// batched GEMMs around an in-place softmax that made the scores do a round trip through memory
// (batched_matmul_qt_k + scale_tensor + softmax + batched_matmul_probs_v, src/transformer.rs:539-550, :877-1121).
//
// One persistent CTA per SM walks the (batch, head) problems:
//   warp 0      TMA producer: Q [128 x dqk] and K [S x dqk] (K-major tiles, 128B swizzle), V [S x dv] (MN-major boxes)
//   warp 1      owns tensor memory (two buffers of [scores 128 cols | output 128 cols]) and issues the MMAs:
//                 scores = Q . K^T  (kind::tf32, M 128, N S), then, once the probabilities are in shared memory,
//                 out = P . V       (M 128, N dv); the score product of problem n+1 is issued before the output
//                 product of problem n, so it runs while the softmax warps work on problem n
//   warps 2-5   one TMEM lane quadrant each, one score row per lane: row maximum (pass 1), exp and row sum with the
//               exponentials written back to tensor memory (pass 2), normalised probabilities into shared memory in
//               the A-operand layout of the second product (pass 3) -- one exp per score; the same shared-memory tile
//               is what a TMA store copies to the caller's probs tensor when the tape wants it; then the output
//               accumulator is drained through the (by then free) probability tile and stored with TMA.
// HBM traffic is Q, K, V in and the output (plus the probabilities only when asked for).  Every mbarrier wait is
// bounded (see mbar_wait): on expiry the CTA raises the error word, drains and frees its tensor memory.
// The fp32-faithful 3xTF32 mode would need hi / lo copies of all four tiles (more shared memory than an SM has at
// S = 128, dqk = 96) and keeps the batched-GEMM route.
#include <cuda.h>

#include "tc_common.cuh"

bool talos_tc_make_operand_map(CUtensorMap* out, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, bool mn_major,
                               int64_t batch, int64_t stride);
bool talos_tc_make_output_map(CUtensorMap* out, const float* base, int64_t slabs, int64_t rows, int64_t cols, int64_t ld, int64_t slab_stride);
bool talos_tc_ready_for(talos_ctx* ctx);

namespace {

struct AttnArgs {
  int BH, S, dqk, dv;
  float scale_log2e;                        // scale * log2(e): the softmax runs on exp2
  int causal, want_probs;
  int32_t* status; unsigned wait_spins;
};

constexpr int ATT_THREADS = 6 * 32;

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) { float e; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x)); return e; }

__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                    const __grid_constant__ CUtensorMap tmap_p, AttnArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int kq = g.dqk / 32, ks = g.S / 32, nv = g.dv / 32;               // k-blocks of the two products, 32-column boxes of V
  const int Q_KB = BM * 128, K_KB = g.S * 128, P_KB = BM * 128, V_KB = nv * 4096;
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kq * Q_KB;
  uint8_t* sV = sK + kq * K_KB;
  uint8_t* sP = sV + ks * V_KB;
  uint64_t* bars = (uint64_t*)(sP + ks * P_KB);
  uint64_t* qk_full = bars;        uint64_t* qk_empty = bars + 1;
  uint64_t* v_full = bars + 2;     uint64_t* v_empty = bars + 3;
  uint64_t* p_full = bars + 4;
  uint64_t* s_full = bars + 5;     // [2] scores of buffer b complete
  uint64_t* o_full = bars + 7;     // [2] output of buffer b complete
  uint64_t* acc_empty = bars + 9;  // [2] both accumulators of buffer b drained
  uint32_t* tmem_slot = (uint32_t*)(bars + 11);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(qk_full, 1); mbar_init(qk_empty, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1); mbar_init(p_full, 4);
    for (int b = 0; b < 2; ++b) { mbar_init(s_full + b, 1); mbar_init(o_full + b, 1); mbar_init(acc_empty + b, 4); }
    abort_flag[0] = 0; abort_flag[1] = (int)g.wait_spins;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int first = blockIdx.x, step = gridDim.x;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      uint32_t ph = 0; bool ok = true;
      for (int bh = first; bh < g.BH && ok; bh += step, ph ^= 1) {
        if (!mbar_wait(qk_empty, ph ^ 1, abort_flag)) break;
        mbar_expect_tx(qk_full, (uint32_t)(kq * (Q_KB + K_KB)));
        for (int kb = 0; kb < kq; ++kb) {
          tma_load_3d(sQ + kb * Q_KB, &tmap_q, kb * 32, 0, bh, qk_full);      // rows past S are filled with zeros
          tma_load_3d(sK + kb * K_KB, &tmap_k, kb * 32, 0, bh, qk_full);
        }
        if (!mbar_wait(v_empty, ph ^ 1, abort_flag)) break;
        mbar_expect_tx(v_full, (uint32_t)(ks * V_KB));
        for (int kb = 0; kb < ks; ++kb)
          for (int j = 0; j < nv; ++j) tma_load_3d(sV + kb * V_KB + j * 4096, &tmap_v, 32 * j, kb * 32, bh, v_full);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(g.S >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((uint32_t)(g.dv >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t ph_qk = 0, ph_pv = 0, acc_ph[2] = {0, 0};
      bool ok = true;
      auto scores = [&](int n) {             // Q . K^T of this CTA's n-th problem into buffer n & 1
        const int b = n & 1;
        if (!mbar_wait(acc_empty + b, acc_ph[b] ^ 1, abort_flag)) { ok = false; return; }
        if (!mbar_wait(qk_full, ph_qk, abort_flag)) { ok = false; return; }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(b * 256);
        for (int kb = 0; kb < kq; ++kb)
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_tf32(d, make_desc(smem_u32(sQ + kb * Q_KB) + k * 32, 16, 1024, 2), make_desc(smem_u32(sK + kb * K_KB) + k * 32, 16, 1024, 2), idesc_s,
                        (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(qk_empty); tc_commit(s_full + b);
        ph_qk ^= 1; acc_ph[b] ^= 1;
      };
      auto output = [&](int n) {             // P . V of the n-th problem
        const int b = n & 1;
        if (!mbar_wait(p_full, ph_pv, abort_flag)) { ok = false; return; }
        if (!mbar_wait(v_full, ph_pv, abort_flag)) { ok = false; return; }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(b * 256 + 128);
        for (int kb = 0; kb < ks; ++kb)
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_tf32(d, make_desc(smem_u32(sP + kb * P_KB) + k * 32, 16, 1024, 2), make_desc(smem_u32(sV + kb * V_KB) + k * 1024, BK * 128, 512, 1), idesc_o,
                        (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(v_empty); tc_commit(o_full + b);
        ph_pv ^= 1;
      };
      const int count = first < g.BH ? (g.BH - first + step - 1) / step : 0;
      if (count > 0) scores(0);
      for (int n = 0; n < count && ok; ++n) {
        if (n + 1 < count) scores(n + 1);
        if (ok) output(n);
      }
    }
  } else {
    // ------------------------------------------------------------- softmax + output: one TMEM lane quadrant per warp, one row per lane
    const int quad = warp & 3, row = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t ph[2] = {0, 0}; bool ok = true; int n = 0; bool stores_pending = false;
    for (int bh = first; bh < g.BH && ok; bh += step, ++n) {
      const int b = n & 1;
      const uint32_t t_s = tmem_base + (uint32_t)(b * 256) + lane_off, t_o = t_s + 128;
      if (!mbar_wait(s_full + b, ph[b], abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int lim = g.causal ? min(row + 1, g.S) : g.S;                // row sees columns [0, lim)
      uint32_t r[32];
      float mx = -INFINITY;
      for (int c = 0; c < ks; ++c) {                                     // pass 1: row maximum
        tmem_ld32(t_s + (uint32_t)(c * 32), r); tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) if (c * 32 + j < lim) mx = fmaxf(mx, __uint_as_float(r[j]));
      }
      const float mxs = mx * g.scale_log2e;
      float sum = 0.f;
      for (int c = 0; c < ks; ++c) {                                     // pass 2: exponentials (kept in tensor memory) and row sum
        tmem_ld32(t_s + (uint32_t)(c * 32), r); tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float e = (c * 32 + j < lim) ? fast_exp2(__uint_as_float(r[j]) * g.scale_log2e - mxs) : 0.f;
          sum += e; r[j] = __float_as_uint(e);
        }
        tmem_st32(t_s + (uint32_t)(c * 32), r);
      }
      tmem_st_wait();
      const float inv = 1.f / sum;
      if (stores_pending) { if (lane == 0) tma_store_wait_read<0>(); __syncwarp(); stores_pending = false; }   // the previous problem's stores still read the tile
      for (int c = 0; c < ks; ++c) {                                     // pass 3: probabilities into the A-operand tile
        tmem_ld32(t_s + (uint32_t)(c * 32), r); tmem_ld_wait();
        float* dst = (float*)(sP + c * P_KB) + row * 32;
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4)
          *(float4*)(dst + ((q4 ^ (lane & 7)) << 2)) = make_float4(__uint_as_float(r[4 * q4]) * inv, __uint_as_float(r[4 * q4 + 1]) * inv,
                                                                  __uint_as_float(r[4 * q4 + 2]) * inv, __uint_as_float(r[4 * q4 + 3]) * inv);
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(p_full);
        if (g.want_probs && quad * 32 < g.S) {                           // (rows past S exist only as padding of the 128-row tile)
          for (int c = 0; c < ks; ++c) tma_store_3d(&tmap_p, sP + c * P_KB + quad * 4096, c * 32, quad * 32, bh);
          tma_store_commit();
        }
      }
      // output accumulator: complete once P . V has retired, which also frees the probability tile for staging
      if (!mbar_wait(o_full + b, ph[b], abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (g.want_probs) { if (lane == 0) tma_store_wait_read<0>(); __syncwarp(); }
      for (int c = 0; c < nv; ++c) {
        tmem_ld32(t_o + (uint32_t)(c * 32), r); tmem_ld_wait();
        float* dst = (float*)(sP + c * P_KB) + row * 32;                 // this warp's 32 rows of tile c: 4 KB, 1024-byte aligned
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4)
          *(float4*)(dst + ((q4 ^ (lane & 7)) << 2)) = make_float4(__uint_as_float(r[4 * q4]), __uint_as_float(r[4 * q4 + 1]), __uint_as_float(r[4 * q4 + 2]),
                                                                  __uint_as_float(r[4 * q4 + 3]));
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (quad * 32 < g.S) {
          for (int c = 0; c < nv; ++c) tma_store_3d(&tmap_o, sP + c * P_KB + quad * 4096, c * 32, quad * 32, bh);
          tma_store_commit();
        }
        mbar_arrive(acc_empty + b);
      }
      stores_pending = true;
      ph[b] ^= 1;
    }
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------- tail
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(g.status, TALOS_DEV_TIMEOUT_BASE + 1800 + (int)blockIdx.x % 100);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace

// Returns false (nothing launched) when the shape is not served: S, dqk, dv multiples of 32; S <= 128; dv <= S;
// 16-byte aligned operands; the four tiles must fit in shared memory.
bool talos_attention_tc_fused(talos_ctx* ctx, const float* q, const float* k, const float* v, float* out, float* probs, int64_t BH,
                              int64_t S, int64_t dqk, int64_t dv, float scale, int causal) {
  if (getenv("TALOS_ATTN_NO_FUSED")) return false;
  if (S < 32 || S > 128 || (S & 31) || (dqk & 31) || (dv & 31) || dqk < 32 || dqk > 128 || dv < 32 || dv > S || BH < 1 || BH >= (1 << 30)) return false;
  if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)probs) & 15) != 0) return false;
  const size_t smem = (size_t)(dqk / 32) * (BM * 128 + S * 128) + (size_t)(S / 32) * ((dv / 32) * 4096 + BM * 128) + 16 * 8 + 1024;
  if (smem > 227 * 1024) return false;
  if (!talos_tc_ready_for(ctx)) return false;
  CUtensorMap tq, tk, tv, to, tp;
  bool ok = talos_tc_make_operand_map(&tq, q, S, dqk, dqk, BM, false, BH, S * dqk) &&
            talos_tc_make_operand_map(&tk, k, S, dqk, dqk, (int)S, false, BH, S * dqk) &&
            talos_tc_make_operand_map(&tv, v, S, dv, dv, BK, true, BH, S * dv) &&
            talos_tc_make_output_map(&to, out, BH, S, dv, dv, S * dv);
  tp = to;
  if (probs) ok = ok && talos_tc_make_output_map(&tp, probs, BH, S, S, S, S * S);
  TALOS_REQUIRE(ok, TALOS_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  AttnArgs g;
  g.BH = (int)BH; g.S = (int)S; g.dqk = (int)dqk; g.dv = (int)dv; g.scale_log2e = scale * 1.4426950408889634f; g.causal = causal; g.want_probs = probs ? 1 : 0;
  g.status = ctx->dev_status; g.wait_spins = ctx->dbg_wait_spins ? ctx->dbg_wait_spins : WAIT_SPINS;
  TALOS_CHECK_CUDA(cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = (int)std::min<int64_t>(BH, ctx->sm_count);
  attention_tc_kernel<<<grid, ATT_THREADS, smem, ctx->stream>>>(tq, tk, tv, to, tp, g);
  talos_launched(ctx, "attention_tc_fused");
  return true;
}
