// Two-CTA tensor-core GEMM (tcgen05 cta_group::2): a cluster of two CTAs computes one 256 x BN output tile.
// Each CTA stages its own 128 rows of A and its own half of the B columns (plain TMA loads, no multicast); the
// leader CTA issues tcgen05.mma.cta_group::2, which reads both CTAs' shared memory and writes 128 accumulator
// rows into each CTA's TMEM.  Per output element this moves a third less operand data from L2 than two
// independent 128 x BN tiles and leaves room for a deeper pipeline (6 stages of 32 KB, or 3 in 3xTF32 mode).
//
// Barriers (same shared-memory offsets in both CTAs):
//   full[s]   TF32: in the leader, armed with both CTAs' bytes; the peer's TMA completes on it through the cluster
//             window.  3xTF32: local, each CTA's own bytes (its converter warps wait on it).
//   conv[s]   in the leader, 8 arrivals (4 converter warps x 2 CTAs).           (3xTF32 only)
//   empty[s]  local, released in both CTAs by one tcgen05.commit with a cluster mask.
//   tfull[a]  local, same commit mechanism.   tempty[a]  in the leader, 16 arrivals (8 epilogue warps x 2 CTAs).
// Every wait is bounded; a CTA that gives up raises the error word and still reaches the closing cluster barrier.
#include "tc_common.cuh"

void talos_splitk_reduce(talos_ctx* ctx, const float* partial, int splits, int64_t M, int64_t N, float* C,
                         int64_t ldc, const EpiArgs& epi);

namespace {

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion may be signalled on the peer CTA's mbarrier (address in the cluster window).
__device__ __forceinline__ void tma_load_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(0) : "memory");   // batch member 0: the pair kernel is not batched
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_mma2_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives (once the MMAs issued so far retire) on the barrier at this offset in BOTH CTAs of the pair.
__device__ __forceinline__ void tc_commit2(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

template <int BN, int STAGES, bool X3, bool A_MN, bool B_MN, bool BPS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(X3 ? 448 : 320, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_b_lo, TcArgs g) {
  constexpr int BH = BN / 2;                                   // B columns staged by each CTA
  constexpr int A_BYTES = BM * BK * 4, B_BYTES = BH * BK * 4;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_BYTES;
  uint8_t* sAlo = sB + STAGES * B_BYTES;
  uint8_t* sBlo = sAlo + (X3 ? STAGES * A_BYTES : 0);
  float* stage_all = (float*)(sBlo + (X3 ? STAGES * B_BYTES : 0));
  uint64_t* bars = (uint64_t*)(stage_all + 8 * 32 * 32);
  uint64_t* full = bars;
  uint64_t* conv = full + STAGES;
  uint64_t* empty = conv + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                     // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(conv + s, 8); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull + a, 1); mbar_init(tempty + a, 16); }
    abort_flag[0] = 0; abort_flag[1] = (int)g.wait_spins;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc2(tmem_slot, TMEM_COLS); tmem_relinquish2(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                              // the peer's barriers exist before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_mn = g.m_tiles * g.n_tiles;                  // m_tiles counts 256-row tiles here
  const int items = tiles_mn * g.splits;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (one per CTA)
    if (lane == 0) {
      prefetch_tmap(&tmap_a); prefetch_tmap(&tmap_b); if (BPS) prefetch_tmap(&tmap_b_lo);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int it = pair; it < items && ok; it += npairs) {
        const int ks = it / tiles_mn, rem = it % tiles_mn; int mb, nb; tc_tile_coords(rem, g.m_tiles, g.n_tiles, g.group_m, mb, nb);
        const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
        const int row0 = mb * 2 * BM + (int)rank * BM, col0 = nb * BN + (int)rank * BH;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort_flag)) { ok = false; break; }
          uint32_t bar;
          if (X3) { mbar_expect_tx(full + stage, A_BYTES + B_BYTES + (BPS ? B_BYTES : 0)); bar = smem_u32(full + stage); }
          else { if (rank == 0) mbar_expect_tx(full + stage, 2 * (A_BYTES + B_BYTES)); bar = map_to_cta(smem_u32(full + stage), 0); }
          uint8_t* a_dst = sA + stage * A_BYTES; uint8_t* b_dst = sB + stage * B_BYTES;
          if (BPS) {
            uint8_t* bl_dst = sBlo + stage * B_BYTES;
            if (B_MN) { for (int j = 0; j < BH / 32; ++j) tma_load_pair(bl_dst + j * (BK * 128), &tmap_b_lo, col0 + 32 * j, kb * BK, bar); }
            else tma_load_pair(bl_dst, &tmap_b_lo, kb * BK, col0, bar);
          }
          if (A_MN) { for (int j = 0; j < BM / 32; ++j) tma_load_pair(a_dst + j * (BK * 128), &tmap_a, row0 + 32 * j, kb * BK, bar); }
          else tma_load_pair(a_dst, &tmap_a, kb * BK, row0, bar);
          if (B_MN) { for (int j = 0; j < BH / 32; ++j) tma_load_pair(b_dst + j * (BK * 128), &tmap_b, col0 + 32 * j, kb * BK, bar); }
          else tma_load_pair(b_dst, &tmap_b, kb * BK, col0, bar);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      const uint32_t a_lbo = A_MN ? BK * 128 : 16, b_lbo = B_MN ? BK * 128 : 16;
      const uint32_t a_kstep = A_MN ? 1024 : UMMA_K * 4, b_kstep = B_MN ? 1024 : UMMA_K * 4;
      const uint32_t a_sbo = A_MN ? 512 : 1024, b_sbo = B_MN ? 512 : 1024, a_lay = A_MN ? 1 : 2, b_lay = B_MN ? 1 : 2;
      int stage = 0; uint32_t phase = 0; int tcount = 0; uint32_t acc_phase[2] = {0, 0}; bool ok = true;
      for (int it = pair; it < items && ok; it += npairs) {
        const int ks = it / tiles_mn;
        const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
        // The item's reduction runs as chains of chain_kb k-blocks: the first chain accumulates into the running
        // buffer, every further one into the other buffer, which the epilogue warps fold into the running one.
        const int run = tcount & 1; ++tcount;
        const int ckb = g.chain_kb > 0 ? g.chain_kb : (kb1 - kb0);
        for (int c0 = kb0; c0 < kb1 && ok; c0 += ckb) {
          const int buf = (c0 == kb0) ? run : (run ^ 1), c1 = min(kb1, c0 + ckb);
          if (!mbar_wait(tempty + buf, acc_phase[buf] ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
          for (int kb = c0; kb < c1; ++kb) {
            if (!mbar_wait((X3 ? conv : full) + stage, phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_hi = smem_u32(sA + stage * A_BYTES), b_hi = smem_u32(sB + stage * B_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint32_t accum = (kb > c0 || k > 0) ? 1u : 0u;
              const uint64_t da = make_desc(a_hi + k * a_kstep, a_lbo, a_sbo, a_lay), db = make_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lay);
              if (X3) {
                const uint32_t a_lo = smem_u32(sAlo + stage * A_BYTES), b_lo = smem_u32(sBlo + stage * B_BYTES);
                const uint64_t dal = make_desc(a_lo + k * a_kstep, a_lbo, a_sbo, a_lay), dbl = make_desc(b_lo + k * b_kstep, b_lbo, b_sbo, b_lay);
                tc_mma2_tf32(d_tmem, dal, db, idesc, accum);
                tc_mma2_tf32(d_tmem, da, dbl, idesc, 1u);
                tc_mma2_tf32(d_tmem, da, db, idesc, 1u);
              } else {
                tc_mma2_tf32(d_tmem, da, db, idesc, accum);
              }
            }
            tc_commit2(empty + stage);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          tc_commit2(tfull + buf);
          acc_phase[buf] ^= 1;
        }
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------- epilogue: each CTA drains its own 128 accumulator rows
    const uint32_t tempty_leader[2] = {map_to_cta(smem_u32(tempty + 0), 0), map_to_cta(smem_u32(tempty + 1), 0)};
    int tcount = 0; uint32_t acc_phase[2] = {0, 0}; bool ok = true; uint32_t store_count = 0;
    for (int it = pair; it < items && ok; it += npairs) {
      const int ks = it / tiles_mn, rem = it % tiles_mn; int mb, nb; tc_tile_coords(rem, g.m_tiles, g.n_tiles, g.group_m, mb, nb);
      const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
      const int run = tcount & 1, other = run ^ 1; ++tcount;
      const int ckb = g.chain_kb > 0 ? g.chain_kb : (kb1 - kb0);
      const uint32_t t_run = tmem_base + (uint32_t)(run * BN), t_other = tmem_base + (uint32_t)(other * BN);
      // first chain: lands in the running buffer; nothing to do but to see it complete
      if (!mbar_wait(tfull + run, acc_phase[run], abort_flag)) { ok = false; break; }
      tc_fence_after();
      // further chains: fold each into the running buffer, then hand its buffer back to the issuer
      for (int c0 = kb0 + ckb; c0 < kb1 && ok; c0 += ckb) {
        if (!mbar_wait(tfull + other, acc_phase[other], abort_flag)) { ok = false; break; }
        tc_fence_after();
        tc_fold_chain<BN>(t_run, t_other, warp);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader[other]);
        acc_phase[other] ^= 1;
      }
      if (!ok) break;
      tc_epilogue_tile<BN>(g, &tmap_c, t_run, warp, lane, stage_all + (warp - 2) * (32 * 32),
                           (long long)mb * 2 * BM + (long long)rank * BM, nb, ks, 0, store_count);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader[run]);
      acc_phase[run] ^= 1;
    }
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  } else if (X3) {
    // ------------------------------------------------------------- converter: splits this CTA's own tiles
    const int ct = threadIdx.x - 320;
    int stage = 0; uint32_t phase = 0; bool ok = true;
    for (int it = pair; it < items && ok; it += npairs) {
      const int ks = it / tiles_mn;
      const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full + stage, phase, abort_flag)) { ok = false; break; }
        float4* ahi = (float4*)(sA + stage * A_BYTES); float4* alo = (float4*)(sAlo + stage * A_BYTES);
        float4* bhi = (float4*)(sB + stage * B_BYTES); float4* blo = (float4*)(sBlo + stage * B_BYTES);
        constexpr int CONV_ITERS = (A_BYTES + (BPS ? 0 : B_BYTES)) / 16 / 128;
#pragma unroll 8
        for (int ci = 0; ci < CONV_ITERS; ++ci) {
          const int i = ct + ci * 128;
          const float4* hi = i < A_BYTES / 16 ? ahi + i : bhi + (i - A_BYTES / 16);
          float4* lo = i < A_BYTES / 16 ? alo + i : blo + (i - A_BYTES / 16);
          *lo = tf32_remainder(*hi);                       // the staged tile itself is the hi operand
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(conv + stage), 0));
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  }

  // ------------------------------------------------------------- tail
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(g.status, TALOS_DEV_TIMEOUT_BASE + 1000 + (int)blockIdx.x % 1000);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync();                                              // neither CTA leaves while the other may still touch its memory
  if (warp == 1) { tc_fence_after(); tmem_dealloc2(tmem_base, TMEM_COLS); }
}

template <int BN, int STAGES, bool X3>
size_t tc2_smem_bytes() {
  return (size_t)STAGES * (BM * BK * 4 + (BN / 2) * BK * 4) * (X3 ? 2 : 1) + 8 * 32 * 32 * 4 + (3 * STAGES + 4) * 8 + 16 + 1024;
}

template <int BN, int STAGES, bool X3, bool A_MN, bool B_MN, bool BPS>
void launch2_one(talos_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tbl, const TcArgs& g, int grid) {
  auto kern = gemm_tc2_kernel<BN, STAGES, X3, A_MN, B_MN, BPS>;
  size_t smem = tc2_smem_bytes<BN, STAGES, X3>();
  TALOS_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, X3 ? 448 : 320, smem, ctx->stream>>>(ta, tb, tc, tbl, g);
  talos_launched(ctx, "gemm_tcgen05_2cta");
}
template <int BN, int STAGES, bool X3, bool BPS>
void launch2_major(talos_ctx* ctx, bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tbl,
                   const TcArgs& g, int grid) {
  if (!a_mn && !b_mn) launch2_one<BN, STAGES, X3, false, false, BPS>(ctx, ta, tb, tc, tbl, g, grid);
  else if (!a_mn && b_mn) launch2_one<BN, STAGES, X3, false, true, BPS>(ctx, ta, tb, tc, tbl, g, grid);
  else if (a_mn && !b_mn) launch2_one<BN, STAGES, X3, true, false, BPS>(ctx, ta, tb, tc, tbl, g, grid);
  else launch2_one<BN, STAGES, X3, true, true, BPS>(ctx, ta, tb, tc, tbl, g, grid);
}

}  // namespace

// Launches the 256 x 256 two-CTA kernel.  `g.m_tiles` must count 256-row tiles; tensor maps as for the one-CTA
// kernel except that the K-major B map has a 128-row box.
void talos_gemm_tc2_launch(talos_ctx* ctx, bool a_mn, bool b_mn, bool x3, bool presplit, const CUtensorMap& ta, const CUtensorMap& tb,
                           const CUtensorMap& tc, const CUtensorMap& tbl, const TcArgs& g, int grid) {
  if (x3 && presplit) launch2_major<256, 3, true, true>(ctx, a_mn, b_mn, ta, tb, tc, tbl, g, grid);
  else if (x3) launch2_major<256, 3, true, false>(ctx, a_mn, b_mn, ta, tb, tc, tbl, g, grid);
  else launch2_major<256, 6, false, false>(ctx, a_mn, b_mn, ta, tb, tc, tbl, g, grid);
}
