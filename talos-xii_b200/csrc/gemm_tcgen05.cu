// Tensor-core GEMM for sm_100a: tcgen05.mma (kind::tf32) with accumulators in TMEM, operands staged
// in 128B-swizzled shared memory by TMA (no multicast), mbarrier pipeline, warp-specialised roles,
// persistent tile loop with a double-buffered TMEM accumulator so the epilogue of one tile overlaps
// the main loop of the next.
//
//   TALOS_MODE_TF32   one TF32 product per term (operands truncated to TF32 by the tensor core).
//   TALOS_MODE_TF32X3 a converter warpgroup splits every fp32 tile in shared memory into
//                     hi = tf32(a) and lo = tf32(a - hi) and the issuer runs lo.hi + hi.lo + hi.hi
//                     into the same accumulator (small terms first): fp32-faithful results.
//
// All four operand layouts are handled by descriptor major-ness (K-major / MN-major), so
// A.B, A.B^T and A^T.B need no transpose pass.  Every wait on an mbarrier is bounded; when one
// gives up the CTA raises an error word, drains, frees its TMEM and returns.
#include <cuda.h>

#include <map>
#include <unordered_map>
#include <mutex>
#include <tuple>
#include <vector>

#include "tc_common.cuh"

void talos_splitk_reduce(talos_ctx* ctx, const float* partial, int splits, int64_t M, int64_t N, float* C,
                         int64_t ldc, const EpiArgs& epi);
void talos_gemm_tc2_launch(talos_ctx* ctx, bool a_mn, bool b_mn, bool x3, bool presplit, const CUtensorMap& ta, const CUtensorMap& tb,
                           const CUtensorMap& tc, const CUtensorMap& tbl, const TcArgs& g, int grid);

namespace {

// Shared storage layout (dynamic, 1024-byte aligned):
//   [STAGES][A tile (hi)] [STAGES][B tile (hi)] ([STAGES][A lo] [STAGES][B lo] in X3 mode) barriers...
// BPS (3xTF32 only): the B operand arrives already split into TF32 hi / lo matrices (two tensor maps), so the
// converter warps only split A.  Used when B is small (weights): it is then split once per call instead of once
// per output tile.
// Warp roles: 0 = TMA producer, 1 = TMEM owner + MMA issuer, then the epilogue warps, then (3xTF32) the converter
// warps.  When both operands are split in the kernel (no pre-split B: the weight-gradient products, whose epilogue
// runs once per 16 k-blocks) the converter is the busy role, so it gets eight warps and the epilogue four.
// EW: epilogue warps when not 0: 16 for the K <= 64 configurations, which are all epilogue (four warps per TMEM lane
// quadrant, one 32-column chunk of a 128-column tile each); 8 for the 256-column tiles that split both operands in the
// kernel (one split-K item per CTA: nothing overlaps its chain fold and partial-tile store).
template <bool X3, bool BPS, int BN = 256, int EW = 0> struct TcRoles {
  // (narrow tiles with a pre-split B are converter-bound too: their epilogue moves 32 or 64 columns a tile)
  static constexpr bool CONV_HEAVY = X3 && (!BPS || BN <= 64);
  static constexpr int EPI_WARPS = EW ? EW : (CONV_HEAVY ? 4 : 8);
  static constexpr int CONV_WARPS = X3 ? (CONV_HEAVY ? 8 : 4) : 0;
  static constexpr int THREADS = (2 + EPI_WARPS + CONV_WARPS) * 32;       // 448 (3xTF32) or 320 (TF32) by default; 576 / 704 with EW = 8 / 16
};

// SBUF: staging buffers per epilogue warp (2 where the configuration leaves the shared memory for it).
// AUXT: the epilogue multiplies by tanh'(saved activation), fetching the activation tiles by TMA (tmap_aux), and
// accumulates the column sums of what it stores (see tc_epilogue_tile_aux).
template <int BN, int STAGES, bool X3, bool A_MN, bool B_MN, int MINB, bool BPS, int SBUF, bool AUXT, int EW = 0>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const CUtensorMap& tmap_c, const CUtensorMap& tmap_b_lo,
                                             const CUtensorMap* tmap_aux, const TcArgs& g) {
  constexpr int A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4;
  // DUAL (3xTF32, 32-column tiles): these products are bound by the NUMBER of MMA instructions (~90 cycles each however
  // narrow), so hi.hi and hi.lo run as ONE 64-column MMA against [B hi | B lo] -- the lo tile sits right behind the hi
  // tile in shared memory -- into a 64-column accumulator whose halves the epilogue warps add: two MMAs per k-step
  // instead of three.
  constexpr bool DUAL = X3 && BN == 32;
  constexpr int ACC_COLS = DUAL ? 2 * BN : BN;
  constexpr int B_STRIDE = DUAL ? 2 * B_BYTES : B_BYTES;             // bytes between the B tiles of consecutive stages
  constexpr uint32_t TMEM_COLS = (2 * ACC_COLS) < 32 ? 32 : (2 * ACC_COLS);
  constexpr int EPI_WARPS = TcRoles<X3, BPS, BN, EW>::EPI_WARPS, CONV_WARPS = TcRoles<X3, BPS, BN, EW>::CONV_WARPS;
  constexpr int STAGE_WARPS = EPI_WARPS > 8 ? EPI_WARPS : 8;        // staging buffers (and AUXT barriers) are laid out for at least eight warps
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_BYTES;
  uint8_t* sAlo = sB + STAGES * B_STRIDE;
  uint8_t* sBlo = DUAL ? sB + B_BYTES : sAlo + (X3 ? STAGES * A_BYTES : 0);
  float* stage_all = (float*)(sAlo + (X3 ? STAGES * A_BYTES : 0) + ((X3 && !DUAL) ? STAGES * B_BYTES : 0));   // one 4 KB block per staging buffer of every epilogue warp (at least eight warps' worth), 1024-byte aligned (TMA-store swizzle)
  uint64_t* bars = (uint64_t*)(stage_all + STAGE_WARPS * 32 * 32 * SBUF);
  uint64_t* aux_bars = bars; bars += AUXT ? STAGE_WARPS : 0;                   // AUXT: one barrier per epilogue warp for its activation tiles
  uint64_t* full = bars;                   // TMA -> (converter | issuer)
  uint64_t* conv = full + STAGES;          // converter -> issuer (X3)
  uint64_t* empty = conv + STAGES;         // issuer (commit) -> TMA
  uint64_t* tfull = empty + STAGES;        // issuer (commit) -> epilogue, per accumulator buffer
  uint64_t* tempty = tfull + 2;            // epilogue -> issuer
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(conv + s, CONV_WARPS ? CONV_WARPS : 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull + a, 1); mbar_init(tempty + a, EPI_WARPS); }
    if (AUXT) for (int w = 0; w < STAGE_WARPS; ++w) mbar_init(aux_bars + w, 1);
    abort_flag[0] = 0; abort_flag[1] = (int)g.wait_spins;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_mn = g.m_tiles * g.n_tiles;
  const int per_batch = tiles_mn * g.splits;              // work items of one batch member
  const int items = per_batch * g.batch;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a); prefetch_tmap(&tmap_b); if (BPS) prefetch_tmap(&tmap_b_lo);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      // L2 prefetch of the streamed operands, PF_DIST k-blocks ahead of the loads along this CTA's own (item, k-block)
      // sequence: with two or three stages in flight the pipeline cannot cover DRAM latency by itself, but it does
      // cover the latency of an L2 hit.
      constexpr int PF_DIST = STAGES + 4;
      int pf_it = blockIdx.x, pf_kb = 0, pf_kb1 = 0, pf_mb = 0, pf_nb = 0, pf_bz = 0;
      auto pf_decode = [&]() {
        if (pf_it >= items) return;
        pf_bz = pf_it / per_batch; const int r = pf_it - pf_bz * per_batch;
        const int ks = r / tiles_mn, rem = r % tiles_mn; tc_tile_coords(rem, g.m_tiles, g.n_tiles, g.group_m, pf_mb, pf_nb);
        pf_kb = ks * g.kb_per_split; pf_kb1 = min(g.kb_total, pf_kb + g.kb_per_split);
      };
      auto pf_step = [&]() {                                   // prefetch the k-block at the look-ahead position, then advance it
        if (pf_it >= items) return;
        if (g.pf_a) {
          if (A_MN) { for (int j = 0; j < BM / 32; ++j) tma_prefetch_3d(&tmap_a, pf_mb * BM + 32 * j, pf_kb * BK, pf_bz); }
          else tma_prefetch_3d(&tmap_a, pf_kb * BK, pf_mb * BM, pf_bz);
        }
        if (g.pf_b) {
          if (B_MN) { for (int j = 0; j < BN / 32; ++j) tma_prefetch_3d(&tmap_b, pf_nb * BN + 32 * j, pf_kb * BK, pf_bz); }
          else tma_prefetch_3d(&tmap_b, pf_kb * BK, pf_nb * BN, pf_bz);
        }
        if (++pf_kb >= pf_kb1) { pf_it += gridDim.x; pf_decode(); }
      };
      const bool pf_on = g.pf_a || g.pf_b;
      const bool b_resident = BPS && g.kb_total <= STAGES && STAGES % g.kb_total == 0 && g.group_m >= g.m_tiles && g.batch == 1 && g.splits == 1;
      int b_loads_left = 0, b_panel = -1;
      if (pf_on) { pf_decode(); for (int i = 0; i < PF_DIST; ++i) pf_step(); }
      for (int it = blockIdx.x; it < items && ok; it += gridDim.x) {
        const int bz = it / per_batch, r = it - bz * per_batch;
        const int ks = r / tiles_mn, rem = r % tiles_mn; int mb, nb; tc_tile_coords(rem, g.m_tiles, g.n_tiles, g.group_m, mb, nb);
        const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (pf_on) pf_step();
          if (!mbar_wait(empty + stage, phase ^ 1, abort_flag)) { ok = false; break; }
          // Test hook: this stage is never armed nor loaded, so its consumers' bounded waits run out and the CTA
          // leaves through the abort path (nothing faults; the loads already in flight land and are ignored).
          if (g.dbg_skip_kb >= 0 && blockIdx.x == 0 && it == 0 && kb - kb0 == g.dbg_skip_kb) { if (++stage == STAGES) { stage = 0; phase ^= 1; } continue; }
          // A product whose k-blocks divide the stage count (K = 32: the input gradient of the fused heads; K = 64 with
          // two stages: the first layer) meets the SAME B tile every time it comes back to a stage for as long as it
          // stays in one column panel, and the plain tile order walks a CTA through one panel after the other: each
          // stage's B buffers are filled on the stage's first use in a panel and kept.
          if (b_resident && kb == kb0 && nb != b_panel) { b_panel = nb; b_loads_left = STAGES; }
          const bool load_b = !b_resident || b_loads_left > 0;
          if (b_resident && b_loads_left > 0) --b_loads_left;
          mbar_expect_tx(full + stage, A_BYTES + (load_b ? B_BYTES + (BPS ? B_BYTES : 0) : 0));
          uint8_t* a_dst = sA + stage * A_BYTES; uint8_t* b_dst = sB + stage * B_STRIDE;
          if (BPS && load_b) {
            uint8_t* bl_dst = sBlo + stage * B_STRIDE;
            if (B_MN) { for (int j = 0; j < BN / 32; ++j) tma_load_3d(bl_dst + j * (BK * 128), &tmap_b_lo, nb * BN + 32 * j, kb * BK, bz, full + stage); }
            else tma_load_3d(bl_dst, &tmap_b_lo, kb * BK, nb * BN, bz, full + stage);
          }
          if (A_MN) { for (int j = 0; j < BM / 32; ++j) tma_load_3d(a_dst + j * (BK * 128), &tmap_a, mb * BM + 32 * j, kb * BK, bz, full + stage); }
          else tma_load_3d(a_dst, &tmap_a, kb * BK, mb * BM, bz, full + stage);
          if (load_b) {
            if (B_MN) { for (int j = 0; j < BN / 32; ++j) tma_load_3d(b_dst + j * (BK * 128), &tmap_b, nb * BN + 32 * j, kb * BK, bz, full + stage); }
            else tma_load_3d(b_dst, &tmap_b, kb * BK, nb * BN, bz, full + stage);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t a_lbo = A_MN ? BK * 128 : 16, b_lbo = B_MN ? BK * 128 : 16;
      const uint32_t a_kstep = A_MN ? 1024 : UMMA_K * 4, b_kstep = B_MN ? 1024 : UMMA_K * 4;
      const uint32_t a_sbo = A_MN ? 512 : 1024, b_sbo = B_MN ? 512 : 1024, a_lay = A_MN ? 1 : 2, b_lay = B_MN ? 1 : 2;
      int stage = 0; uint32_t phase = 0; int tcount = 0; uint32_t acc_phase[2] = {0, 0}; bool ok = true;
      for (int it = blockIdx.x; it < items && ok; it += gridDim.x) {
        const int ks = (it % per_batch) / tiles_mn;
        const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
        // The item's reduction runs as chains of chain_kb k-blocks (the whole item when chain_kb = 0): the first chain
        // accumulates into the item's running buffer, every further one into the other buffer, which the epilogue warps
        // fold into the running one -- the fp32-faithful mode keeps its accumulation chains short that way without
        // sending partial tiles through memory.
        const int run = tcount & 1; ++tcount;
        const int ckb = g.chain_kb > 0 ? g.chain_kb : (kb1 - kb0);
        for (int c0 = kb0; c0 < kb1 && ok; c0 += ckb) {
          const int buf = (c0 == kb0) ? run : (run ^ 1), c1 = min(kb1, c0 + ckb);
          if (!mbar_wait(tempty + buf, acc_phase[buf] ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * ACC_COLS);
          for (int kb = c0; kb < c1; ++kb) {
            // 3xTF32: the products that need no converted operand (hi.hi, and hi.lo when B arrives pre-split) are issued
            // as soon as the loads have landed, beside the converter; the rest once the lo tiles are written.
            const bool early = X3 && g.early_pass && !(DUAL && !BPS);    // (DUAL without a pre-split B has nothing to start early)
            if (!mbar_wait((X3 && !early ? conv : full) + stage, phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_hi = smem_u32(sA + stage * A_BYTES), b_hi = smem_u32(sB + stage * B_STRIDE);
            const uint32_t a_lo = smem_u32(sAlo + stage * A_BYTES), b_lo = smem_u32(sBlo + stage * B_STRIDE);
            if (DUAL) {
              const uint32_t idesc2 = (idesc & ~(0x3Fu << 17)) | ((uint32_t)(ACC_COLS >> 3) << 17);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)                                                                 // hi.[hi | lo]
                tc_mma_tf32(d_tmem, make_desc(a_hi + k * a_kstep, a_lbo, a_sbo, a_lay), make_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lay), idesc2,
                            (kb > c0 || k > 0) ? 1u : 0u);
              if (early) { if (!mbar_wait(conv + stage, phase, abort_flag)) { ok = false; break; } tc_fence_after(); }
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)                                                                 // lo.hi
                tc_mma_tf32(d_tmem, make_desc(a_lo + k * a_kstep, a_lbo, a_sbo, a_lay), make_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lay), idesc, 1u);
            } else if (early) {
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t da = make_desc(a_hi + k * a_kstep, a_lbo, a_sbo, a_lay), db = make_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lay);
                tc_mma_tf32(d_tmem, da, db, idesc, (kb > c0 || k > 0) ? 1u : 0u);                                  // hi.hi
                if (BPS) tc_mma_tf32(d_tmem, da, make_desc(b_lo + k * b_kstep, b_lbo, b_sbo, b_lay), idesc, 1u);    // hi.lo
              }
              if (!mbar_wait(conv + stage, phase, abort_flag)) { ok = false; break; }
              tc_fence_after();
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t dal = make_desc(a_lo + k * a_kstep, a_lbo, a_sbo, a_lay), db = make_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lay);
                tc_mma_tf32(d_tmem, dal, db, idesc, 1u);                                                            // lo.hi
                if (!BPS) tc_mma_tf32(d_tmem, make_desc(a_hi + k * a_kstep, a_lbo, a_sbo, a_lay), make_desc(b_lo + k * b_kstep, b_lbo, b_sbo, b_lay), idesc, 1u);
              }
            } else {
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint32_t accum = (kb > c0 || k > 0) ? 1u : 0u;
                const uint64_t da = make_desc(a_hi + k * a_kstep, a_lbo, a_sbo, a_lay), db = make_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lay);
                if (X3) {
                  const uint64_t dal = make_desc(a_lo + k * a_kstep, a_lbo, a_sbo, a_lay), dbl = make_desc(b_lo + k * b_kstep, b_lbo, b_sbo, b_lay);
                  tc_mma_tf32(d_tmem, dal, db, idesc, accum);      // lo.hi
                  tc_mma_tf32(d_tmem, da, dbl, idesc, 1u);         // hi.lo
                  tc_mma_tf32(d_tmem, da, db, idesc, 1u);          // hi.hi
                } else {
                  tc_mma_tf32(d_tmem, da, db, idesc, accum);
                }
              }
            }
            tc_commit(empty + stage);                            // frees the stage when these MMAs retire
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          tc_commit(tfull + buf);                                // chain complete
          acc_phase[buf] ^= 1;
        }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------------------------------------- epilogue: normally 8 warps, two per TMEM lane quadrant,
    // each taking half of the tile's columns (the epilogue is latency-bound per warp, so it needs the extra warps).
    int tcount = 0; uint32_t acc_phase[2] = {0, 0}; bool ok = true; uint32_t store_count = 0;
    TcAuxState aux_st{0u, {0.f, 0.f, 0.f, 0.f}};
    float* const my_stage = stage_all + (warp - 2) * (32 * 32 * SBUF); uint64_t* const aux_bar = aux_bars + (warp - 2);
    if (AUXT && (int)blockIdx.x < items && lane == 0) {        // the first chunk's saved-activation tile, into the first staging buffer
      int mb0, nb0; tc_tile_coords((int)blockIdx.x % tiles_mn, g.m_tiles, g.n_tiles, g.group_m, mb0, nb0);
      tc_aux_request(tmap_aux, my_stage, aux_bar, nb0 * BN + ((warp - 2) >> 2) * (BN / (EPI_WARPS / 4)), (long long)mb0 * BM + (warp & 3) * 32);
    }
    for (int it = blockIdx.x; it < items && ok; it += gridDim.x) {
      const int bz = it / per_batch, r = it - bz * per_batch;
      const int ks = r / tiles_mn, rem = r % tiles_mn; int mb, nb; tc_tile_coords(rem, g.m_tiles, g.n_tiles, g.group_m, mb, nb);
      const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
      const int run = tcount & 1, other = run ^ 1; ++tcount;
      const int ckb = g.chain_kb > 0 ? g.chain_kb : (kb1 - kb0);
      const uint32_t t_run = tmem_base + (uint32_t)(run * ACC_COLS), t_other = tmem_base + (uint32_t)(other * ACC_COLS);
      if (!mbar_wait(tfull + run, acc_phase[run], abort_flag)) { ok = false; break; }        // first chain: lands in the running buffer
      tc_fence_after();
      for (int c0 = kb0 + ckb; c0 < kb1 && ok; c0 += ckb) {                                   // further chains: fold, hand the buffer back
        if (!mbar_wait(tfull + other, acc_phase[other], abort_flag)) { ok = false; break; }
        tc_fence_after();
        tc_fold_chain<ACC_COLS, EPI_WARPS>(t_run, t_other, warp);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty + other);
        acc_phase[other] ^= 1;
      }
      if (!ok) break;
      if (DUAL) tc_fold_chain<BN, EPI_WARPS>(t_run, t_run + (uint32_t)BN, warp);       // (hi.hi + lo.hi) += hi.lo
      if constexpr (AUXT) {
        const int nit = it + (int)gridDim.x; int nmb = 0, nnb = 0;
        if (nit < items) tc_tile_coords(nit % tiles_mn, g.m_tiles, g.n_tiles, g.group_m, nmb, nnb);
        if (!tc_epilogue_tile_aux<BN, SBUF, EPI_WARPS>(g, &tmap_c, tmap_aux, t_run, warp, lane, my_stage, aux_bar, abort_flag,
                                            (long long)mb * BM, nb, nit < items, (long long)nmb * BM, nnb, store_count, aux_st)) { ok = false; break; }
      } else {
        tc_epilogue_tile<BN, EPI_WARPS, SBUF>(g, &tmap_c, t_run, warp, lane, my_stage, (long long)mb * BM, nb, ks, bz, store_count);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty + run);
      acc_phase[run] ^= 1;
    }
    if (lane == 0) tma_store_wait_read<0>();                 // shared memory must outlive the stores that read it
    __syncwarp();
    if (AUXT && g.colsum_part) {
      // this warp's column sums over all the tiles of the CTA: one partial row per (CTA, lane quadrant); a warp owns
      // half of the columns of each panel, zero where it had no tile
      float* row = g.colsum_part + ((size_t)blockIdx.x * 4 + (warp & 3)) * g.N;
      const int half = (warp - 2) >> 2; constexpr int PART_COLS = BN / (EPI_WARPS / 4), CHUNKS = PART_COLS / 32;
#pragma unroll
      for (int j = 0; j < 4; ++j) {                            // j = (column panel) * CHUNKS + (32-column chunk of this warp's share)
        const int col = (j / CHUNKS) * BN + half * PART_COLS + (j % CHUNKS) * 32 + lane;
        if ((j / CHUNKS) < g.n_tiles && col < g.N) row[col] = aux_st.acc[j];
      }
    }
  } else if (X3) {
    // ------------------------------------------------------------- converter warps: fp32 -> (hi, lo) TF32 pair
    constexpr int CONV_THREADS = (CONV_WARPS ? CONV_WARPS : 1) * 32;
    const int ct = threadIdx.x - (2 + EPI_WARPS) * 32;         // 0 .. CONV_THREADS-1
    int stage = 0; uint32_t phase = 0; bool ok = true;
    for (int it = blockIdx.x; it < items && ok; it += gridDim.x) {
      const int ks = (it % per_batch) / tiles_mn;
      const int kb0 = ks * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full + stage, phase, abort_flag)) { ok = false; break; }
        // The split is elementwise, so it is oblivious to the swizzle: same offset in, same offset out.
        float4* ahi = (float4*)(sA + stage * A_BYTES); float4* alo = (float4*)(sAlo + stage * A_BYTES);
        float4* bhi = (float4*)(sB + stage * B_STRIDE); float4* blo = (float4*)(sBlo + stage * B_STRIDE);
        constexpr int CONV_ITERS = (A_BYTES + (BPS ? 0 : B_BYTES)) / 16 / CONV_THREADS;
        static_assert((A_BYTES + (BPS ? 0 : B_BYTES)) % (16 * CONV_THREADS) == 0, "tile bytes must divide evenly over the converter threads");
#pragma unroll 8
        for (int ci = 0; ci < CONV_ITERS; ++ci) {
          const int i = ct + ci * CONV_THREADS;
          const float4* hi = i < A_BYTES / 16 ? ahi + i : bhi + (i - A_BYTES / 16);
          float4* lo = i < A_BYTES / 16 ? alo + i : blo + (i - A_BYTES / 16);
          *lo = tf32_remainder(*hi);                       // the staged tile itself is the hi operand
        }
        fence_proxy_async();                                   // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(conv + stage);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  }

  // ------------------------------------------------------------- tail
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up: report it, give copies still in flight time to land, then release TMEM.
    if (threadIdx.x == 0) atomicExch(g.status, TALOS_DEV_TIMEOUT_BASE + (int)blockIdx.x % 1000);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

template <int BN, int STAGES, bool X3, bool A_MN, bool B_MN, int MINB = 1, bool BPS = false, int SBUF = 1, int EW = 0>
__global__ void __launch_bounds__((TcRoles<X3, BPS, BN, EW>::THREADS), MINB)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_b_lo, const __grid_constant__ TcArgs g) {
  gemm_tc_body<BN, STAGES, X3, A_MN, B_MN, MINB, BPS, SBUF, false, EW>(tmap_a, tmap_b, tmap_c, tmap_b_lo, nullptr, g);
}
// The fused input-gradient configurations (prepared weights, both operands K-major): one more tensor map.  3xTF32 with the
// pre-split weights (two stages), or TF32 with the rounded weights (three stages).
template <int BN, int STAGES, bool X3, int SBUF, int EW = 0>
__global__ void __launch_bounds__((TcRoles<X3, X3, BN, EW>::THREADS), 1)
gemm_tc_aux_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c,
                   const __grid_constant__ CUtensorMap tmap_b_lo, const __grid_constant__ CUtensorMap tmap_aux, const __grid_constant__ TcArgs g) {
  gemm_tc_body<BN, STAGES, X3, false, false, 1, X3, SBUF, true, EW>(tmap_a, tmap_b, tmap_c, tmap_b_lo, &tmap_aux, g);
}

// Dense copy of a [rows][cols] matrix (pitch ld) rounded to TF32 with round-to-nearest.  In the fast TF32
// mode the tensor core TRUNCATES its fp32 inputs, a bias of ~3.5e-4 per operand; pre-rounding the small operand
// (the weights) removes its half of that bias for a few microseconds of extra work.
__global__ void round_tf32_kernel(const float* __restrict__ in, long long ld, int rows, int cols, int out_ld, float* __restrict__ out) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * out_ld) return;
  int r = (int)(idx / out_ld), c = (int)(idx % out_ld);
  out[idx] = c < cols ? __uint_as_float(cvt_tf32(in[(long long)r * ld + c])) : 0.f;
}

// Dense TF32 hi / lo copies of a [rows][cols] matrix: hi = rna(a), lo = rna(a - hi).
__global__ void split_tf32_kernel(const float* __restrict__ in, long long ld, int rows, int cols, int out_ld, float* __restrict__ hi,
                                  float* __restrict__ lo) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * out_ld) return;
  int r = (int)(idx / out_ld), c = (int)(idx % out_ld);
  float a = c < cols ? in[(long long)r * ld + c] : 0.f;
  float h = __uint_as_float(cvt_tf32(a));
  hi[idx] = h; lo[idx] = __uint_as_float(cvt_tf32(a - h));
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr; cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// Encoded tensor maps are kept per thread, keyed on everything that goes into them: a training loop calls the same
// products on the same buffers every step, and cuTensorMapEncodeTiled costs about a microsecond of host time per map
// (three or four maps per product).  A map holds no reference to the memory it describes, so a stale entry for a
// buffer that was freed and reallocated with the same address and shape is still the right map.
struct TmapKey {
  const void* base; int64_t a, b, c, d, e; int kind;
  bool operator==(const TmapKey& o) const { return base == o.base && a == o.a && b == o.b && c == o.c && d == o.d && e == o.e && kind == o.kind; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = (uint64_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ULL;
    for (int64_t v : {k.a, k.b, k.c, k.d, k.e, (int64_t)k.kind}) h = (h ^ (uint64_t)v) * 0x100000001B3ULL + (h >> 29);
    return (size_t)h;
  }
};
bool tmap_cached(const TmapKey& key, CUtensorMap* out, bool (*encode)(const TmapKey&, CUtensorMap*)) {
  thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  if (!encode(key, out)) return false;
  if (cache.size() >= 512) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// 3-D fp32 tensor map over `batch` row-major [rows][cols] matrices (cols contiguous) `stride` elements apart,
// box = [1][box_rows][32 cols].  A plain GEMM is a batch of one.  Rows past the end of a batch member are filled
// with zeros by the copy engine, never read from the next member.
bool encode_operand_map(const TmapKey& k, CUtensorMap* out) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const int64_t rows = k.a, cols = k.b, ld = k.c, batch = k.d, stride = k.e; const int box_rows = k.kind >> 1; const bool mn_major = k.kind & 1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * sizeof(float), (cuuint64_t)stride * sizeof(float)};
  cuuint32_t box[3] = {32u, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)k.base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}
bool make_tmap(CUtensorMap* out, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, bool mn_major,
               int64_t batch = 1, int64_t stride = 0) {
  if (batch <= 1) { batch = 1; stride = rows * ld; }
  return tmap_cached(TmapKey{base, rows, cols, ld, batch, stride, (box_rows << 1) | (mn_major ? 1 : 0)}, out, encode_operand_map);
}

// 3-D fp32 tensor map for results: [slabs][rows][cols], box = [1][32][32], 128B swizzle.  C itself is one
// slab; split-K partial sums are `splits` dense slabs; a batched product has one slab per batch member,
// `slab_stride` elements apart.  Stores are clipped per slab by the map.
bool encode_output_map(const TmapKey& k, CUtensorMap* out) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const int64_t slabs = k.a, rows = k.b, cols = k.c, ld = k.d, slab_stride = k.e;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)slabs};
  cuuint64_t strides[2] = {(cuuint64_t)ld * sizeof(float), (cuuint64_t)slab_stride * sizeof(float)};
  cuuint32_t box[3] = {32u, 32u, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)k.base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}
bool make_out_tmap(CUtensorMap* out, const float* base, int64_t slabs, int64_t rows, int64_t cols, int64_t ld, int64_t slab_stride) {
  return tmap_cached(TmapKey{base, slabs, rows, cols, ld, slab_stride, -1}, out, encode_output_map);
}

template <int BN, int STAGES, bool X3, int SBUF = 1, int EW = 0>
size_t tc_smem_bytes() {
  return (size_t)STAGES * (BM * BK * 4 + BN * BK * 4) * (X3 ? 2 : 1) + (EW > 8 ? EW : 8) * 32 * 32 * 4 * SBUF + (3 * STAGES + 4) * 8 + 16 + 1024;
}

template <int BN, int STAGES, bool X3, bool A_MN, bool B_MN, int MINB = 1, bool BPS = false, int SBUF = 1, int EW = 0>
void launch_one(talos_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tbl, const TcArgs& g, int grid) {
  auto kern = gemm_tc_kernel<BN, STAGES, X3, A_MN, B_MN, MINB, BPS, SBUF, EW>;
  size_t smem = tc_smem_bytes<BN, STAGES, X3, SBUF, EW>();
  TALOS_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, TcRoles<X3, BPS, BN, EW>::THREADS, smem, ctx->stream>>>(ta, tb, tc, tbl, g);
  talos_launched(ctx, "gemm_tcgen05");
}

template <int BN, int STAGES, bool X3, int MINB = 1, bool BPS = false, int SBUF = 1, int EW = 0>
void launch_major(talos_ctx* ctx, bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tbl,
                  const TcArgs& g, int grid) {
  if (!a_mn && !b_mn) launch_one<BN, STAGES, X3, false, false, MINB, BPS, SBUF, EW>(ctx, ta, tb, tc, tbl, g, grid);
  else if (!a_mn && b_mn) launch_one<BN, STAGES, X3, false, true, MINB, BPS, SBUF, EW>(ctx, ta, tb, tc, tbl, g, grid);
  else if (a_mn && !b_mn) launch_one<BN, STAGES, X3, true, false, MINB, BPS, SBUF, EW>(ctx, ta, tb, tc, tbl, g, grid);
  else launch_one<BN, STAGES, X3, true, true, MINB, BPS, SBUF, EW>(ctx, ta, tb, tc, tbl, g, grid);
}

static inline bool x3_mode(int mode) { return mode == TALOS_MODE_TF32X3; }
thread_local bool g_check_fold = false;   // set by the self-check: the whole reduction in one item, so that its 17 k-blocks are two chains folded on chip
thread_local bool g_check_pair = false;   // set by the start-up self-check so that its short reduction still exercises the pair kernel

// A batched product: `batch` independent GEMMs whose operands are `stride*` elements apart (batch 1: a plain GEMM).
struct TcBatch { int64_t batch, stride_a, stride_b, stride_c; };

void tc_launch(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
               int64_t ldb, float* C, int64_t ldc, int mode, const EpiArgs& epi, const TcBatch& bt = TcBatch{1, 0, 0, 0},
               const TcExtra* extra = nullptr) {
  const bool batched = bt.batch > 1;
  const bool b_given = extra && extra->b_hi && !batched && (x3_mode(mode) ? extra->b_lo != nullptr : true);
  const bool a_mn = (opA == TALOS_OP_T), b_mn = (opB == TALOS_OP_N), x3 = (mode == TALOS_MODE_TF32X3);
  int bn = N > 128 ? 256 : N > 64 ? 128 : N > 32 ? 64 : 32;
  // Short reductions with a prepared small B (K <= 64: the first layer's forward product) are all epilogue: 128-column
  // tiles leave the shared memory for two staging buffers per epilogue warp, so that the store engine's read of one
  // chunk overlaps the arithmetic of the next.
  const bool short_k = !batched && x3 && bn == 256 && K <= 64 && (b_given || (opB == TALOS_OP_N ? K * N : N * K) <= (1 << 20)) && !getenv("TALOS_TC_NO_SHORTK");
  if (short_k) bn = 128;
  // (that configuration is all epilogue: sixteen epilogue warps, one 32-column chunk of a tile each, instead of eight with two)
  const bool wide_epi = short_k && !getenv("TALOS_TC_NO_WIDE_EPI");
  TcArgs g;
  g.M = (int)M; g.N = (int)N; g.K = (int)K; g.C = C; g.ldc = ldc; g.epi = epi; g.status = ctx->dev_status; g.partial = nullptr;
  g.batch = (int)std::max<int64_t>(bt.batch, 1); g.stride_c = batched ? bt.stride_c : 0;
  g.early_pass = getenv("TALOS_TC_NO_EARLY") ? 0 : 1;
  g.wait_spins = ctx->dbg_wait_spins ? ctx->dbg_wait_spins : WAIT_SPINS; g.dbg_skip_kb = ctx->dbg_skip_kb;
  // Streamed K-major operands (more than 8 MB, i.e. not something that stays in L2 anyway) of the 3xTF32 kernels are
  // prefetched into L2 ahead of the loads: those kernels have only two or three stages in flight.  Measured on
  // 65 536 x 256 x 256: 3xTF32 A.B 65.0 -> 59.7 us, A.B^T 63.4 -> 59.3 us; the TF32 kernels (four or more stages)
  // and MN-major operands (one prefetch per 32-column box) got slower with it, so they do not use it.
  {
    const bool pf_off = getenv("TALOS_TC_NO_PREFETCH") != nullptr;
    g.pf_a = (!pf_off && x3 && !a_mn && (int64_t)M * K * g.batch > (2 << 20)) ? 1 : 0;
    g.pf_b = (!pf_off && x3 && !b_mn && (int64_t)N * K * g.batch > (2 << 20)) ? 1 : 0;
  }
  // 256-wide outputs with at least 256 rows and a long reduction run on CTA pairs (cta_group::2): 256 x 256 tiles
  // halve the operand bytes each SM has to pull per flop.  For short reductions (K = 256: 8 k-blocks a tile) the
  // pair's start-up and cross-CTA hand-offs cost more than that saves (measured 8 % slower at K = 256, 10 % faster
  // at K = 2048), so those stay on the one-CTA kernel.
  // They also need enough 256 x 256 tiles to occupy every CTA pair without splitting K (the split-K weight-gradient
  // shapes have one or two tiles and are faster on 148 independent CTAs than on 74 pairs).
  const bool pair_shape = K >= 1024 && ceil_div(M, 2 * BM) * ceil_div(N, 256) >= ctx->sm_count / 2;
  const bool pair = ctx->dbg_skip_kb < 0 && !batched && bn == 256 && M >= 256 && (pair_shape || g_check_pair || getenv("TALOS_TC_FORCE_PAIR")) && !getenv("TALOS_TC_NO_PAIR");
  g.m_tiles = (int)ceil_div(M, pair ? 2 * BM : BM); g.n_tiles = (int)ceil_div(N, bn); g.kb_total = (int)ceil_div(K, BK);
  // Groups of 8 row panels once there are enough tiles for the order to matter (with ~148 tiles in flight an 8-wide
  // group makes each wave touch 8 row panels and ~n/8 column panels instead of every row panel).
  g.group_m = (g.m_tiles >= 16 && g.n_tiles >= 4 && !getenv("TALOS_TC_NO_RASTER")) ? 8 : g.m_tiles;
  int tiles = g.m_tiles * g.n_tiles, splits = 1;
  const int workers = pair ? ctx->sm_count / 2 : ctx->sm_count;   // CTAs, or CTA pairs
  // Split K when the output tiles alone cannot occupy the workers.  The tensor core truncates when it adds into the
  // fp32 accumulator, a bias that grows with the length of the accumulation chain (measured ~7e-9 relative per k
  // element), so the fp32-faithful mode never chains more than 512 k elements in TMEM: longer reductions MUST be split
  // there, and the partial sums are added in fp32 (round-to-nearest) by the reduction kernel.
  // The split count is chosen per number of rounds r (every worker runs r items): splits = r * workers / tiles, and
  // the cheapest r * (k-blocks per item + a few k-blocks' worth of per-item pipeline fill and epilogue) wins -- e.g. the
  // 256 x 256 x 65 536 weight gradient runs 2 x 147 items of 14 k-blocks on 148 CTAs instead of 2 x 128 of 16.
  const int cap = (x3 && !batched) ? 512 / BK : g.kb_total;     // (batched products with K > 512 are not routed here)
  // The one-CTA kernel, too, meets the chain cap on chip (a finished chain is folded into a running sum in the second
  // TMEM buffer), so an item may hold several chains: the 256 x 256 x 65 536 weight gradient then runs 2 x 74 items of 28
  // k-blocks (two chains) instead of 2 x 147 of 14, which halves the partial tiles the gather kernel has to add.
  const bool fold_one = x3 && !batched && !pair && !getenv("TALOS_TC_NO_FOLD");
  g.kb_per_split = g.kb_total;
  if (!batched && ((tiles * 2 <= workers && g.kb_total >= 16) || g.kb_total > cap)) {
    const int item_overhead = 3;
    long long best_cost = -1;
    for (int r = 1; r <= 8; ++r) {
      const int s_r = (int)std::max<int64_t>(1, (int64_t)r * workers / tiles);
      int kps = (int)ceil_div(g.kb_total, s_r);
      if (kps < 8 && r > 1) break;                                  // items would become shorter than their own overhead
      kps = std::max(kps, std::min(8, g.kb_total));
      if (kps > cap && !(fold_one && kps <= 8 * cap)) continue;
      const int chains = (int)ceil_div(kps, cap);
      const long long cost = (long long)ceil_div((int64_t)tiles * ceil_div(g.kb_total, kps), workers) * (kps + item_overhead + (chains - 1));
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; g.kb_per_split = kps; }
    }
    if (g.kb_per_split > cap && !(fold_one && best_cost >= 0)) g.kb_per_split = cap;
  }
  if (g_check_fold && fold_one && g.kb_total > cap) g.kb_per_split = g.kb_total;
  g.chain_kb = (fold_one && g.kb_per_split > cap) ? cap : 0;
  if (pair && x3 && g.kb_total > cap && !getenv("TALOS_TC_NO_FOLD")) {
    // CTA-pair kernel: the chain cap is met ON CHIP (finished chains are folded into a running sum in TMEM), so K is
    // split through memory only as far as it takes to keep the pairs busy: the smallest power-of-two split whose
    // last round is at least 95 % full (4096^3: 2 slabs of 4 chains instead of 8 slabs through memory).
    int best_s = 1; double best_eff = 0.0;
    for (int s_ext = 1; s_ext <= 8 && g.kb_total / s_ext >= cap; s_ext *= 2) {
      const int64_t n_items = (int64_t)tiles * s_ext, rounds = ceil_div(n_items, workers);
      const double eff = (double)n_items / (double)(rounds * workers);
      if (eff > best_eff + 0.03) { best_eff = eff; best_s = s_ext; }
      if (eff >= 0.95) break;
    }
    g.kb_per_split = (int)(ceil_div(ceil_div(g.kb_total, best_s), cap) * cap);     // whole chains per item
    g.chain_kb = cap;
  }
  splits = (int)ceil_div(g.kb_total, g.kb_per_split);
  g.splits = splits;
  // kernel-level scratch: [split-K partials][TF32-rounded copy of the small operand]
  const int64_t a_rows = a_mn ? K : M, a_cols = a_mn ? M : K, b_rows = b_mn ? K : N, b_cols = b_mn ? N : K;
  const int64_t a_elems = a_rows * a_cols, b_elems = b_rows * b_cols;
  const bool round_a = !batched && !x3 && !b_given && a_elems <= b_elems && a_elems <= (1 << 20);
  const bool round_b = !batched && !x3 && !b_given && !round_a && b_elems <= (1 << 20);
  const int64_t r_rows = round_a ? a_rows : b_rows, r_cols = round_a ? a_cols : b_cols, r_ld = (r_cols + 3) & ~int64_t(3);
  const bool plain_epi = !epi.bias && !epi.aux_out && !epi.aux_in && !epi.act && !epi.beta;    // the reduction kernel applies the epilogue
  const bool keep_partials = extra && extra->partial && splits > 1 && plain_epi && extra->partial_floats >= (size_t)splits * M * N;
  if (extra && extra->splits_out) *extra->splits_out = keep_partials ? splits : 1;
  const size_t partial_bytes = (splits > 1 && !keep_partials) ? ((sizeof(float) * (size_t)splits * M * N + 255) & ~size_t(255)) : 0;
  const bool presplit = !batched && x3 && (b_given || b_elems <= (1 << 20));
  const int64_t s_ld = (b_cols + 3) & ~int64_t(3);
  const size_t round_bytes = (round_a || round_b) ? sizeof(float) * (size_t)(r_rows * r_ld) : (presplit && !b_given) ? 2 * sizeof(float) * (size_t)(b_rows * s_ld) : 0;
  char* scratch = (partial_bytes + round_bytes) ? (char*)talos_workspace(ctx, partial_bytes + round_bytes) : nullptr;
  if (splits > 1) g.partial = keep_partials ? extra->partial : (float*)scratch;
  const float* B_lo = nullptr;
  if (b_given) {                       // prepared by the caller: same shape and pitch as B
    B = extra->b_hi; B_lo = x3 ? extra->b_lo : nullptr;
  } else if (presplit) {
    float* hi = (float*)(scratch + partial_bytes); float* lo = hi + b_rows * s_ld;
    split_tf32_kernel<<<(unsigned)ceil_div(b_rows * s_ld, 256), 256, 0, ctx->stream>>>(B, ldb, (int)b_rows, (int)b_cols, (int)s_ld, hi, lo);
    talos_launched(ctx, "split_tf32");
    B = hi; B_lo = lo; ldb = s_ld;
  }
  if (round_a || round_b) {
    float* dst = (float*)(scratch + partial_bytes);
    round_tf32_kernel<<<(unsigned)ceil_div(r_rows * r_ld, 256), 256, 0, ctx->stream>>>(round_a ? A : B, round_a ? lda : ldb, (int)r_rows, (int)r_cols, (int)r_ld, dst);
    talos_launched(ctx, "round_tf32");
    if (round_a) { A = dst; lda = r_ld; } else { B = dst; ldb = r_ld; }
  }

  CUtensorMap ta, tb;
  bool ok = a_mn ? make_tmap(&ta, A, K, M, lda, BK, true, bt.batch, bt.stride_a) : make_tmap(&ta, A, M, K, lda, BM, false, bt.batch, bt.stride_a);
  const int b_box_rows = pair ? bn / 2 : bn;                      // each CTA of a pair stages half of the B columns
  ok = ok && (b_mn ? make_tmap(&tb, B, K, N, ldb, BK, true, bt.batch, bt.stride_b) : make_tmap(&tb, B, N, K, ldb, b_box_rows, false, bt.batch, bt.stride_b));
  CUtensorMap tbl = tb;
  if (presplit) ok = ok && (b_mn ? make_tmap(&tbl, B_lo, K, N, ldb, BK, true) : make_tmap(&tbl, B_lo, N, K, ldb, b_box_rows, false));
  // Results leave through TMA stores when the destination is 16-byte aligned with a 16-byte pitch, N is a
  // multiple of 4 (a TMA store clips the innermost axis in 16-byte units, so a ragged N would spill into the
  // pitch padding) and the epilogue does not also save the pre-activation; otherwise through direct stores.
  CUtensorMap tc = ta;
  g.tma_out = 0;
  const bool both = epi.act != 0 && epi.aux_in != nullptr && epi.dact != 0;
  const bool epi_aligned = !(((uintptr_t)epi.bias) & 15) && !(((uintptr_t)epi.aux_in) & 15) && !(epi.ld_aux_in & 3);
  if (splits > 1) { if (!(N & 3)) { g.tma_out = 1; ok = ok && make_out_tmap(&tc, g.partial, splits, M, N, N, M * N); } }
  else if (!(((uintptr_t)C) & 15) && !(ldc & 3) && !(N & 3) && !(batched && (bt.stride_c & 3)) && !epi.aux_out && !both && epi_aligned) {
    g.tma_out = 1; ok = ok && make_out_tmap(&tc, C, g.batch, M, N, ldc, batched ? bt.stride_c : M * ldc);
  }
  if (extra && extra->colsum_slabs_out) *extra->colsum_slabs_out = 0;
  g.colsum_part = nullptr;
  int grid = (int)std::min<int64_t>((int64_t)tiles * splits * g.batch, ctx->sm_count);
  // The input gradient of a tanh layer takes tanh' and the bias gradient's column sums into its epilogue: the K <= 64
  // configuration (128-column tiles, two staging buffers) and the 256-column one (a single staging buffer).
  const bool aux_x3 = presplit && (short_k || bn == 256), aux_tf32 = !x3 && b_given && bn == 256;
  const bool aux_cfg = (aux_x3 || aux_tf32) && !batched && !a_mn && !b_mn && !pair && splits == 1 && g.n_tiles * (bn / 64) <= 4;
  const bool auxt = extra && extra->tanh_saved && extra->colsum_part && extra->colsum_slabs_out && aux_cfg && !(N & 31) && plain_epi && g.tma_out &&
                    !(((uintptr_t)extra->tanh_saved) & 15) && !(extra->ld_saved & 3) && extra->colsum_floats >= (size_t)4 * grid * N &&
                    !getenv("TALOS_TC_NO_FUSED_DACT");
  CUtensorMap tx = tc;
  if (auxt) ok = ok && make_out_tmap(&tx, extra->tanh_saved, 1, M, N, extra->ld_saved, M * extra->ld_saved);
  TALOS_REQUIRE(ok, TALOS_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  if (auxt) {
    g.colsum_part = extra->colsum_part;
#define TALOS_TC_AUX(BNv, ST, X3v, SB, EWv)                                                                                         \
  { const size_t smem = tc_smem_bytes<BNv, ST, X3v, SB, EWv>() + 128;                                                               \
    TALOS_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc_aux_kernel<BNv, ST, X3v, SB, EWv>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    gemm_tc_aux_kernel<BNv, ST, X3v, SB, EWv><<<grid, TcRoles<X3v, X3v, BNv, EWv>::THREADS, smem, ctx->stream>>>(ta, tb, tc, tbl, tx, g); }
    if (!x3) TALOS_TC_AUX(256, 3, false, 2, 0)
    else if (bn == 128 && wide_epi) TALOS_TC_AUX(128, 2, true, 1, 16)
    else if (bn == 128) TALOS_TC_AUX(128, 2, true, 2, 0)
    else TALOS_TC_AUX(256, 2, true, 1, 0)
#undef TALOS_TC_AUX
    talos_launched(ctx, "gemm_tcgen05");
    *extra->colsum_slabs_out = 4 * grid;
    return;
  }
  if (pair) {
    talos_gemm_tc2_launch(ctx, a_mn, b_mn, x3, presplit, ta, tb, tc, tbl, g, 2 * std::min(tiles * splits, workers));
    if (splits > 1 && !keep_partials) talos_splitk_reduce(ctx, g.partial, splits, M, N, C, ldc, epi);
    return;
  }
  // (tile width, stages and staging buffers per epilogue warp in TF32 mode, the same for the 3xTF32 kernels)
#define TALOS_TC_CASE(BNv, ST, SB, ST3, SB3)                                                                      \
  if (bn == BNv) {                                                                                                \
    if (x3 && presplit) launch_major<BNv, ST3, true, 1, true, SB3>(ctx, a_mn, b_mn, ta, tb, tc, tbl, g, grid);    \
    else if (x3 && BNv == 256 && !getenv("TALOS_TC_NO_EPI8")) launch_major<BNv, ST3, true, 1, false, SB3, (BNv == 256 ? 8 : 0)>(ctx, a_mn, b_mn, ta, tb, tc, tb, g, grid); \
    else if (x3) launch_major<BNv, ST3, true, 1, false, SB3>(ctx, a_mn, b_mn, ta, tb, tc, tb, g, grid);           \
    else launch_major<BNv, ST, false, 1, false, SB>(ctx, a_mn, b_mn, ta, tb, tc, tb, g, grid);                    \
  }
  if (short_k && presplit && wide_epi) launch_major<128, 2, true, 1, true, 1, 16>(ctx, a_mn, b_mn, ta, tb, tc, tbl, g, grid);
  else if (short_k && presplit) launch_major<128, 2, true, 1, true, 2>(ctx, a_mn, b_mn, ta, tb, tc, tbl, g, grid);
  else TALOS_TC_CASE(256, 3, 2, 2, 1) else TALOS_TC_CASE(128, 6, 1, 3, 1) else TALOS_TC_CASE(64, 8, 1, 4, 1) else TALOS_TC_CASE(32, 8, 2, 4, 2)
#undef TALOS_TC_CASE
  if (splits > 1 && !keep_partials) talos_splitk_reduce(ctx, g.partial, splits, M, N, C, ldc, epi);
}

// Start-up self-check: every operand layout in both modes against the fp32 CUDA-core kernel on a
// shape with ragged edges.  Any mismatch or device-side timeout disables the tensor-core path for
// this context (the fp32 kernel then serves all modes) instead of returning wrong numbers.
// With batch > 1 the LD x LD buffers are cut into `batch` members of LD / batch rows each (M, N, K must fit).
bool self_check_shape(talos_ctx* ctx, const int M, const int N = 328, const int K = 296, const int batch = 1) {
  const int LD = 520, member_rows = LD / batch;
  const int64_t stride = (int64_t)member_rows * LD;
  const TcBatch bt{batch, stride, stride, stride};
  size_t elems = (size_t)LD * LD;
  float *A = nullptr, *B = nullptr, *C0 = nullptr, *C1 = nullptr;
  std::vector<float> h(elems), r0(elems), r1(elems);
  uint64_t s = 0x243F6A8885A308D3ULL;
  for (auto& v : h) { s = s * 6364136223846793005ULL + 1442695040888963407ULL; v = (float)((double)(s >> 11) / 9007199254740992.0 * 2.0 - 1.0); }
  bool pass = true;
  const bool dbg = getenv("TALOS_DEBUG") != nullptr;
  try {
    TALOS_CHECK_CUDA(cudaMalloc(&A, elems * 4)); TALOS_CHECK_CUDA(cudaMalloc(&B, elems * 4));
    TALOS_CHECK_CUDA(cudaMalloc(&C0, elems * 4)); TALOS_CHECK_CUDA(cudaMalloc(&C1, elems * 4));
    TALOS_CHECK_CUDA(cudaMemcpyAsync(A, h.data(), elems * 4, cudaMemcpyHostToDevice, ctx->stream));
    TALOS_CHECK_CUDA(cudaMemcpyAsync(B, h.data() + 17, (elems - 17) * 4, cudaMemcpyHostToDevice, ctx->stream));
    EpiArgs e{nullptr, nullptr, 0, nullptr, 0, 0, 0, 0};
    for (int opA = 0; opA < 2 && (pass || dbg); ++opA)
      for (int opB = 0; opB < 2 && (pass || dbg); ++opB) {
        TALOS_CHECK_CUDA(cudaMemsetAsync(C0, 0, elems * 4, ctx->stream));
        talos_gemm_fp32_launch(ctx, opA, opB, M, N, K, A, LD, stride, B, LD, stride, C0, LD, stride, batch, e);
        TALOS_CHECK_CUDA(cudaMemcpyAsync(r0.data(), C0, elems * 4, cudaMemcpyDeviceToHost, ctx->stream));
        for (int mode = TALOS_MODE_TF32X3; mode <= TALOS_MODE_TF32 && (pass || dbg); ++mode) {
          TALOS_CHECK_CUDA(cudaMemsetAsync(C1, 0, elems * 4, ctx->stream));
          tc_launch(ctx, opA, opB, M, N, K, A, LD, B, LD, C1, LD, mode, e, bt);
          TALOS_CHECK_CUDA(cudaMemcpyAsync(r1.data(), C1, elems * 4, cudaMemcpyDeviceToHost, ctx->stream));
          TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
          int32_t st = 0; TALOS_CHECK_CUDA(cudaMemcpy(&st, ctx->dev_status, 4, cudaMemcpyDeviceToHost));
          if (dbg) fprintf(stderr, "[talos self-check] opA=%d opB=%d mode=%d status=%d\n", opA, opB, mode, st);
          if (st != 0) { cudaMemset(ctx->dev_status, 0, 64); pass = false; if (!dbg) break; }
          double num = 0, den = 0;
          for (int bz = 0; bz < batch; ++bz)
            for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) {
              const size_t i = ((size_t)bz * member_rows + m) * LD + n;
              double d = (double)r1[i] - r0[i]; num += d * d; den += (double)r0[i] * r0[i];
            }
          double rel = sqrt(num / (den > 0 ? den : 1));
          if (dbg) fprintf(stderr, "[talos self-check]   rel err %.3e  c[0]=%g ref %g c[last]=%g ref %g\n", rel, r1[0], r0[0], r1[(size_t)(M - 1) * LD + N - 1], r0[(size_t)(M - 1) * LD + N - 1]);
          bool good = rel <= (mode == TALOS_MODE_TF32 ? 2e-3 : 8e-6);   // (a wrong layout or a lost k-block shows as 1e-3 or more; the mode's contract is 1e-5)
          if (!good) { pass = false; if (dbg) { good = true; continue; } }
          for (int m = 0; m < LD && pass; ++m)                                               // nothing outside any member's [M,N]
            for (int n = ((m % member_rows) < M && m / member_rows < batch ? N : 0); n < LD; ++n) if (r1[(size_t)m * LD + n] != 0.f) { pass = false; break; }
        }
      }
  } catch (const talos_error&) { pass = false; cudaGetLastError(); }
  cudaStreamSynchronize(ctx->stream);
  cudaFree(A); cudaFree(B); cudaFree(C0); cudaFree(C1);
  return pass;
}

// Rows 200: one-CTA kernels; rows 456: the CTA-pair kernel (two 256-row tiles, the second one ragged; once more with a
// reduction longer than one accumulation chain); then a batch
// of three small ragged products (tiles must neither read nor write across batch members).
bool self_check(talos_ctx* ctx) {
  bool ok = self_check_shape(ctx, 200) && self_check_shape(ctx, 72, 88, 104, 3);
  g_check_fold = true;
  ok = ok && self_check_shape(ctx, 200, 328, 520);                               // K = 520 in one item on the one-CTA kernel: two chains, folded on chip
  g_check_fold = false;
  g_check_pair = true;
  ok = ok && self_check_shape(ctx, 456) && self_check_shape(ctx, 456, 328, 520);   // K = 520: two chains, folded on chip in 3xTF32 mode
  g_check_pair = false;
  return ok;
}

}  // namespace

static bool tc_ready(talos_ctx* ctx) {
  if (ctx->tc_state < 0) return false;
  if (getenv("TALOS_DISABLE_TENSOR_CORES")) return false;
  if (ctx->tc_state == 0) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(ctx->stream, &cap);
    if (cap != cudaStreamCaptureStatusNone) return false;      // cannot self-check inside a capture
    ctx->tc_state = self_check(ctx) ? 1 : -1;
  }
  return ctx->tc_state > 0;
}

// For the other tensor-core kernels of the library (the fused attention): the same tensor maps and the same start-up check.
bool talos_tc_make_operand_map(CUtensorMap* out, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, bool mn_major,
                               int64_t batch, int64_t stride) { return make_tmap(out, base, rows, cols, ld, box_rows, mn_major, batch, stride); }
bool talos_tc_make_output_map(CUtensorMap* out, const float* base, int64_t slabs, int64_t rows, int64_t cols, int64_t ld, int64_t slab_stride) {
  return make_out_tmap(out, base, slabs, rows, cols, ld, slab_stride);
}
bool talos_tc_ready_for(talos_ctx* ctx) { return tc_ready(ctx); }

bool talos_gemm_tc_launch(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                          const float* B, int64_t ldb, float* C, int64_t ldc, int mode, const EpiArgs& epi, const TcExtra* extra) {
  if (extra && extra->splits_out) *extra->splits_out = 1;
  if (ctx->tc_state < 0) return false;
  // TMA needs 16-byte aligned bases and row pitches; tiny problems are launch-bound and stay on CUDA cores.
  if ((((uintptr_t)A | (uintptr_t)B) & 15) || (lda & 3) || (ldb & 3) || K < 1) return false;
  if (M * N * K < (1LL << 18) || M < 1 || N < 1) return false;
  if (!tc_ready(ctx)) return false;
  if (extra && extra->b_hi && ((((uintptr_t)extra->b_hi | (uintptr_t)extra->b_lo) & 15) != 0)) return false;
  tc_launch(ctx, opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode, epi, TcBatch{1, 0, 0, 0}, extra);
  return true;
}

// Batched product on the one-CTA kernel: the batch index is the third coordinate of every tensor map, so a tile
// never reads or writes across batch members.  Needs 16-byte aligned strides on top of the plain GEMM's
// conditions; a 3xTF32 product with K > 512 would need split-K and is left to the fp32 kernel.
bool talos_gemm_tc_launch_batched(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                                  int64_t strideA, const float* B, int64_t ldb, int64_t strideB, float* C, int64_t ldc, int64_t strideC,
                                  int64_t batch, int mode, const EpiArgs& epi) {
  if (ctx->tc_state < 0) return false;
  if ((((uintptr_t)A | (uintptr_t)B) & 15) || (lda & 3) || (ldb & 3) || (strideA & 3) || (strideB & 3) || K < 1) return false;
  if (M < 1 || N < 1 || batch < 1 || M * N * K * batch < (1LL << 18) || M * N * K < (1LL << 12)) return false;
  if (mode == TALOS_MODE_TF32X3 && K > 512) return false;
  if (ceil_div(M, BM) * ceil_div(N, 32) * batch >= (1LL << 30)) return false;
  if (!tc_ready(ctx)) return false;
  tc_launch(ctx, opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode, epi, TcBatch{batch, strideA, strideB, strideC});
  return true;
}
