// Device-side building blocks shared by the tensor-core GEMM kernels: PTX wrappers (mbarrier, TMA, tcgen05,
// TMEM), shared-memory matrix descriptors, the fused epilogue helpers and the kernel argument block.
#pragma once
#include <cuda.h>

#include "common.cuh"

// Kernel argument block of the tensor-core GEMM kernels (shared by the one-CTA and CTA-pair launchers).
struct TcArgs {
  int M, N, K;
  int m_tiles, n_tiles, splits, kb_total, kb_per_split;
  float* C; long long ldc;
  float* partial;                          // [splits][M][N] when splits > 1
  EpiArgs epi;
  int32_t* status;
  int tma_out;                             // 1: results leave through TMA stores (tmap_c), 0: direct stores
  int pf_a, pf_b;                          // prefetch this operand's tiles into L2 a few k-blocks ahead (large streamed operands only)
  int chain_kb;                            // CTA-pair 3xTF32 kernel: k-blocks per accumulation chain folded on chip (0: one chain per item)
  int batch;                               // independent problems (third coordinate of every tensor map); 1 for a plain GEMM
  long long stride_c;                      // elements between consecutive batch members of C
  float* colsum_part;                      // AUXT kernels: [4 * grid][N] per-warp-quadrant column sums of the stored result (bias gradient)
  int early_pass;                          // 3xTF32: issue the products of unconverted operands before the converter is done
  int group_m;                             // tile order: m-tiles are walked in groups of this many per column sweep (L2 reuse); >= m_tiles: plain order
  unsigned wait_spins;                     // poll limit of every bounded wait (WAIT_SPINS unless a test shortened it)
  int dbg_skip_kb;                         // test hook: CTA 0's producer never loads this k-block of its first item (-1: off)
};

namespace {

constexpr int BM = 128;                 // tile rows = TMEM lanes
constexpr int BK = 32;                  // fp32 per 128-byte swizzle row
constexpr int UMMA_K = 8;               // K per tcgen05.mma.kind::tf32
constexpr uint32_t WAIT_SPINS = 1u << 22;

// Output-tile order.  Tile `rem` of the m_tiles x n_tiles grid: the m index runs fastest inside a group of `group_m`
// row panels, then the column panel advances, then the next group starts -- so the tiles in flight at any time (one
// per CTA, consecutive `rem`) cover a near-square block of the result and re-use each other's operand panels in L2,
// instead of every wave streaming all of A.
__device__ __forceinline__ void tc_tile_coords(int rem, int m_tiles, int n_tiles, int group_m, int& mb, int& nb) {
  if (group_m >= m_tiles) { nb = rem / m_tiles; mb = rem - nb * m_tiles; return; }
  const int gsz = group_m * n_tiles, grp = rem / gsz, first_m = grp * group_m;
  const int gm = min(group_m, m_tiles - first_m), within = rem - grp * gsz;
  nb = within / gm; mb = first_m + within - nb * gm;
}

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after raising *abort_flag) when the barrier never flips or when
// another role has already given up.
// abort_flag[1] holds the poll limit (set at kernel start from TcArgs::wait_spins); it is read only after the first
// poll has failed, so the common case costs nothing extra.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint32_t limit = (uint32_t)abort_flag[1];
  for (uint32_t i = 1; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    // try_wait itself parks the thread for a hardware-defined interval, so the loop is not hot; back off with
    // nanosleep only when the wait is clearly long (the epilogue waiting out a whole main loop, or a stall).
    if (i > 64 && (i & 63) == 0) { if (*abort_flag) return false; if (i > (1u << 14)) __nanosleep(128); }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Operand tiles: every operand map is [batch][rows][cols]; c2 selects the batch member (0 for a plain GEMM).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Ask the copy engine to bring one box of a tensor map into L2 (no shared-memory destination, no completion signal).
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N_PENDING>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N_PENDING) : "memory"); }
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// 16-column forms for the on-chip fold of accumulation chains (running sum += finished chain, both in TMEM).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                 "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Round to TF32 (10 mantissa bits), nearest with ties away from zero -- the semantics of cvt.rna.tf32.f32 -- with two
// integer operations on the bit pattern (add half an ulp of the kept part to the magnitude, clear the 13 dropped
// bits); the conversion instruction itself issues at a fraction of the integer rate and was the converter warps'
// bottleneck.  A carry out of the mantissa correctly bumps the exponent; Inf/NaN inputs are not expected here.
__device__ __forceinline__ uint32_t cvt_tf32(float x) { return (__float_as_uint(x) + 0x1000u) & 0xFFFFE000u; }

// 3xTF32 split of four staged fp32 values.  The tensor core reads an fp32 word as TF32 by dropping its low 13 bits
// (measured: the error of a plain TF32 product matches truncation, and the split below reproduces the fp32 product to
// 1.8e-6), so the staged tile already IS the hi operand and nothing is written back for it; lo is the remainder
// against that truncation, rounded to TF32.  hi + lo reproduces the value to 2^-21 relative.
__device__ __forceinline__ float4 tf32_remainder(float4 v) {
  float4 l;
  l.x = __uint_as_float(cvt_tf32(v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u)));
  l.y = __uint_as_float(cvt_tf32(v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u)));
  l.z = __uint_as_float(cvt_tf32(v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u)));
  l.w = __uint_as_float(cvt_tf32(v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u)));
  return l;
}

// Shared-memory matrix descriptor for a swizzled operand tile (1024-byte aligned).
//  K-major : layout 2 (128B swizzle, 16-byte atoms): rows of 128 B, 8-row groups 1024 B apart (SBO);
//            the leading offset is unused (1).
//  MN-major: fp32 operands must use layout 1 (128B swizzle with 32-byte atoms, 4-row period):
//            32-float column chunks, each [BK rows][128 B]; chunk stride (LBO) = BK*128 B,
//            4-row k-groups 512 B apart (SBO).  TMA writes it with SWIZZLE_128B_ATOM_32B.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;                  // descriptor version for this architecture
  d |= (uint64_t)layout << 61;
  return d;
}


// Epilogue over one transposed 32x32 staging tile: lane = column, loop over rows.  The activation
// and derivative kinds are template parameters so the row loop carries no per-element branches.
template <int ACT, int DACT>
__device__ __forceinline__ void epilogue_rows_t(const EpiArgs& e, const float* stage, int lane, long long m0, int rows_valid,
                                                long long n, bool col_ok, float* C, long long ldc) {
  const float bias_v = (e.bias && col_ok) ? __ldg(e.bias + n) : 0.f;
#pragma unroll 4
  for (int rr = 0; rr < rows_valid; ++rr) {
    if (!col_ok) continue;
    const long long m = m0 + rr;
    float v = stage[rr * 32 + (lane ^ rr)] + bias_v;
    if (e.aux_out) e.aux_out[m * e.ld_aux_out + n] = v;
    if (ACT) v = talos_act(v, ACT);
    if (DACT) v *= talos_dact(__ldg(e.aux_in + m * e.ld_aux_in + n), DACT);
    if (e.beta) v += C[m * ldc + n];
    C[m * ldc + n] = v;
  }
}
// (EpiArgs by value: a reference would force the kernel's whole argument struct out of the constant bank into a
// local-memory copy, and every field read of every epilogue chunk with it.)
__device__ __noinline__ void epilogue_rows(const EpiArgs e, const float* stage, int lane, long long m0, int rows_valid, long long n,
                                           bool col_ok, float* C, long long ldc) {
  const int dact = e.aux_in ? e.dact : 0;
  switch (e.act * 4 + dact) {
#define TALOS_EPI_CASE(A, D) case (A) * 4 + (D): epilogue_rows_t<A, D>(e, stage, lane, m0, rows_valid, n, col_ok, C, ldc); break;
    TALOS_EPI_CASE(0, 0) TALOS_EPI_CASE(0, 1) TALOS_EPI_CASE(0, 2) TALOS_EPI_CASE(0, 3)
    TALOS_EPI_CASE(1, 0) TALOS_EPI_CASE(1, 1) TALOS_EPI_CASE(1, 2) TALOS_EPI_CASE(1, 3)
    TALOS_EPI_CASE(2, 0) TALOS_EPI_CASE(2, 1) TALOS_EPI_CASE(2, 2) TALOS_EPI_CASE(2, 3)
    TALOS_EPI_CASE(3, 0) TALOS_EPI_CASE(3, 1) TALOS_EPI_CASE(3, 2) TALOS_EPI_CASE(3, 3)
#undef TALOS_EPI_CASE
    default: break;
  }
}

// Fused epilogue on one group of four consecutive columns of one accumulator row.  Everything is a
// named scalar or a float4 (no arrays), so the accumulator values never leave registers.  The host
// guarantees 16-byte alignment of every operand on this path.
template <int ACT, int DACT>
__device__ __forceinline__ float4 epilogue_group(float4 v, const float* __restrict__ bias, const float* __restrict__ aux_in,
                                                 const float* __restrict__ c_old) {
  if (bias) { const float4 b = __ldg((const float4*)bias); v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
  if (ACT) { v.x = talos_act(v.x, ACT); v.y = talos_act(v.y, ACT); v.z = talos_act(v.z, ACT); v.w = talos_act(v.w, ACT); }
  if (DACT) {
    const float4 a = __ldg((const float4*)aux_in);
    v.x *= talos_dact(a.x, DACT); v.y *= talos_dact(a.y, DACT); v.z *= talos_dact(a.z, DACT); v.w *= talos_dact(a.w, DACT);
  }
  if (c_old) { const float4 o = *(const float4*)c_old; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
  return v;
}



// On-chip fold of one finished accumulation chain into the running sum: run[lane][col] += acc[lane][col] in fp32
// (round to nearest), for this warp's TMEM lane quadrant and column half.  This is how the fp32-faithful mode keeps its
// accumulation chains short (the tensor core truncates when it adds into the accumulator) without sending partial
// tiles through memory.
template <int BN, int EPI_WARPS = 8>
__device__ __forceinline__ void tc_fold_chain(uint32_t t_run, uint32_t t_acc, int warp) {
  constexpr int PARTS = EPI_WARPS / 4;                       // warps per TMEM lane quadrant: each takes BN / PARTS columns
  const int quad = warp & 3, half = (warp - 2) >> 2;
  constexpr int HALF_COLS = (PARTS > 1 && BN / PARTS >= 32) ? BN / PARTS : BN;
  const uint32_t row = (uint32_t)(quad * 32) << 16;
#pragma unroll 1
  for (int c0 = half * HALF_COLS; c0 < (half + 1) * HALF_COLS && c0 < BN; c0 += 16) {
    uint32_t a[16], r[16];
    tmem_ld16(t_acc + row + (uint32_t)c0, a);
    tmem_ld16(t_run + row + (uint32_t)c0, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(a[j]));
    tmem_st16(t_run + row + (uint32_t)c0, r);
  }
  tmem_st_wait();
}

// One epilogue warp's share of a finished 128 x BN accumulator: warp w (2..9) owns TMEM lane quadrant w%4 (32 rows,
// one per lane) and half of the columns, drained 32 columns at a time.  `t_base` is the TMEM address of the
// accumulator's first column, `m_base` the global row of TMEM lane 0, `stage` this warp's 4 KB staging buffer.
// SBUF staging buffers per warp (consecutive 4 KB blocks at `stage`): with two, the store engine may still be reading
// the previous chunk while the next one is written.
template <int BN, int EPI_WARPS = 8, int SBUF = 1>
__device__ __forceinline__ void tc_epilogue_tile(const TcArgs& g, const CUtensorMap* tmap_c, uint32_t t_base, int warp, int lane, float* stage,
                                                 long long m_base, int nb, int ks, int bz, uint32_t& store_count) {
  static_assert(EPI_WARPS == 16 || EPI_WARPS == 8 || EPI_WARPS == 4, "four, two or one warp per TMEM lane quadrant");
  float* const c_base = g.C + (long long)bz * g.stride_c;   // this batch member's C (split-K never batches: ks or bz is 0)
  // Each warp drains its 32-lane quadrant (one accumulator row per lane) 32 columns at a time.
  constexpr int PARTS = EPI_WARPS / 4;
  const int quad = warp & 3, half = (warp - 2) >> 2;          // (which of the quadrant's PARTS column shares)
  const long long m0 = m_base + quad * 32;
  const uint32_t t_row = t_base + ((uint32_t)(quad * 32) << 16);
  const int rows_valid = (int)min((long long)32, (long long)g.M - m0);
  constexpr int HALF_COLS = (PARTS > 1 && BN / PARTS >= 32) ? BN / PARTS : BN;
  const int c_begin = half * HALF_COLS, c_end = min((half + 1) * HALF_COLS, BN);
  if (rows_valid <= 0) return;
  if (g.tma_out) {
    // Results leave through TMA stores.  The wait for the previous chunk's TMA store (which is still reading the
    // staging buffer) comes AFTER this chunk's epilogue arithmetic, just before the buffer is overwritten, so the
    // store engine's read overlaps the arithmetic.  (Also keeping the next chunk's TMEM load in flight during the
    // arithmetic was tried: 64 live accumulator registers made every variant spill.)
    int c0 = c_begin;
    bool have = c0 < c_end && (long long)nb * BN + c0 < g.N;
#pragma unroll 1
    while (have) {
      const long long n0 = (long long)nb * BN + c0;
      uint32_t r[32];
      tmem_ld32(t_row + (uint32_t)c0, r);
      tmem_ld_wait();
      const int c1 = c0 + 32;
      const bool have_next = c1 < c_end && (long long)nb * BN + c1 < g.N;
      // Fused epilogue in registers, then a 128B-swizzled 32x32 tile in shared memory that one
      // lane hands to the TMA store engine (clipped to [M,N] by the tensor map).
      float* buf = stage + (SBUF == 2 ? (store_count & 1u) * (32 * 32) : 0);
      {
        const bool fuse = (g.splits == 1) && (lane < rows_valid);
        const long long m = m0 + lane;
        const int dact = g.epi.aux_in ? g.epi.dact : 0;
        const float* bias_p = (fuse && g.epi.bias) ? g.epi.bias + n0 : nullptr;
        const float* aux_p = (fuse && dact) ? g.epi.aux_in + m * g.epi.ld_aux_in + n0 : nullptr;
        const float* cold_p = (fuse && g.epi.beta) ? c_base + m * g.ldc + n0 : nullptr;
        const int groups = (int)min((long long)8, (g.N - n0) >> 2);     // N is a multiple of 4 on this path
#define TALOS_EPI_MATH(A, D)                                                                                            \
  _Pragma("unroll") for (int c = 0; c < 8; ++c) {                                                                      \
if (fuse && c < groups) {                                                                                           \
  float4 v = make_float4(__uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]), __uint_as_float(r[4 * c + 2]),  \
                         __uint_as_float(r[4 * c + 3]));                                                           \
  v = epilogue_group<A, D>(v, bias_p ? bias_p + 4 * c : nullptr, aux_p ? aux_p + 4 * c : nullptr,                  \
                           cold_p ? cold_p + 4 * c : nullptr);                                                      \
  r[4 * c] = __float_as_uint(v.x); r[4 * c + 1] = __float_as_uint(v.y); r[4 * c + 2] = __float_as_uint(v.z);        \
  r[4 * c + 3] = __float_as_uint(v.w);                                                                              \
}                                                                                                                   \
  }
        // The common forward epilogue (bias and / or activation on a full 32-column chunk, nothing read per element)
        // runs WITHOUT per-group conditions on every lane -- rows past M hold garbage the TMA store clips anyway -- so
        // the 32 independent activation chains of a lane can be interleaved instead of running four at a time between
        // branches.
        const bool straight = g.splits == 1 && groups == 8 && !dact && !g.epi.beta && (g.epi.act || g.epi.bias);
#define TALOS_EPI_STRAIGHT(A, HAS_BIAS)                                                                                 \
  { const float4* bp = (const float4*)(g.epi.bias + n0);                                                                \
    _Pragma("unroll") for (int c = 0; c < 8; ++c) {                                                                    \
      const float4 b4 = HAS_BIAS ? __ldg(bp + c) : make_float4(0.f, 0.f, 0.f, 0.f);                                     \
      r[4 * c] = __float_as_uint(talos_act(__uint_as_float(r[4 * c]) + b4.x, A));                                       \
      r[4 * c + 1] = __float_as_uint(talos_act(__uint_as_float(r[4 * c + 1]) + b4.y, A));                               \
      r[4 * c + 2] = __float_as_uint(talos_act(__uint_as_float(r[4 * c + 2]) + b4.z, A));                               \
      r[4 * c + 3] = __float_as_uint(talos_act(__uint_as_float(r[4 * c + 3]) + b4.w, A));                               \
    } }
        if (straight) {
          switch (g.epi.act * 2 + (g.epi.bias ? 1 : 0)) {
            case 2: TALOS_EPI_STRAIGHT(1, false) break;
            case 3: TALOS_EPI_STRAIGHT(1, true) break;
            case 4: TALOS_EPI_STRAIGHT(2, false) break;
            case 5: TALOS_EPI_STRAIGHT(2, true) break;
            case 6: TALOS_EPI_STRAIGHT(3, false) break;
            case 7: TALOS_EPI_STRAIGHT(3, true) break;
            default: TALOS_EPI_STRAIGHT(0, true) break;
          }
        } else
        switch (fuse ? g.epi.act * 4 + dact : 0) {
          case 1: TALOS_EPI_MATH(0, 1) break;
          case 2: TALOS_EPI_MATH(0, 2) break;
          case 3: TALOS_EPI_MATH(0, 3) break;
          case 4: TALOS_EPI_MATH(1, 0) break;
          case 8: TALOS_EPI_MATH(2, 0) break;
          case 12: TALOS_EPI_MATH(3, 0) break;
          default: if (g.epi.bias || g.epi.beta) { TALOS_EPI_MATH(0, 0) } break;
        }
#undef TALOS_EPI_MATH
#undef TALOS_EPI_STRAIGHT
      }
      if (store_count >= SBUF) { if (lane == 0) tma_store_wait_read<SBUF - 1>(); __syncwarp(); }
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *(float4*)(buf + lane * 32 + ((c ^ (lane & 7)) << 2)) =
            make_float4(__uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]), __uint_as_float(r[4 * c + 2]), __uint_as_float(r[4 * c + 3]));
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) { tma_store_3d(tmap_c, buf, (int)n0, (int)m0, ks + bz); tma_store_commit(); }
      ++store_count;
      c0 = c1; have = have_next;
    }
    return;
  }
#pragma unroll 1
  for (int c0 = c_begin; c0 < c_end; c0 += 32) {
    const long long n0 = (long long)nb * BN + c0;
    if (n0 >= g.N) break;                                   // uniform across the warp
    uint32_t r[32];
    tmem_ld32(t_row + (uint32_t)c0, r);
    tmem_ld_wait();
    {
      // Unaligned output: transpose through a padded tile so lanes run along the contiguous axis.
#pragma unroll
      for (int j = 0; j < 32; ++j) stage[lane * 32 + (j ^ lane)] = __uint_as_float(r[j]);    // XOR-swizzled transpose tile
      __syncwarp();
      const long long n = n0 + lane;
      const bool col_ok = n < g.N;
      if (g.splits > 1) {
        float* P = g.partial + ((long long)ks * g.M + m0) * g.N + n;
#pragma unroll 4
        for (int rr = 0; rr < rows_valid; ++rr) if (col_ok) P[(long long)rr * g.N] = stage[rr * 32 + (lane ^ rr)];
      } else {
        epilogue_rows(g.epi, stage, lane, m0, rows_valid, n, col_ok, c_base, g.ldc);
      }
      __syncwarp();
    }
  }
}


// Column sums of a 32 x 32 chunk held one row per lane (r[j] = column j of this lane's row): after five exchange rounds
// lane j holds the sum of column j over the 32 rows.  Each round halves the values a lane keeps: it gives the half that
// belongs to its partner's columns and adds the partner's contribution to its own half (31 shuffles in all).
__device__ __forceinline__ float tc_chunk_colsum(const uint32_t (&r)[32], int lane) {
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float lo = __uint_as_float(r[i]), hi = __uint_as_float(r[i + 16]);
    const bool up = lane & 16;
    const float keep = up ? hi : lo, send = up ? lo : hi;
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int w = 8; w >= 1; w >>= 1) {
#pragma unroll
    for (int i = 0; i < w; ++i) {
      const bool up = lane & w;
      const float keep = up ? v[i + w] : v[i], send = up ? v[i] : v[i + w];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, w);
    }
  }
  return v[0];
}

// Epilogue of the hidden-layer input gradient, fused: result = accumulator * (1 - h^2), and the column sums of the
// result (the bias gradient) accumulated in registers across all the tiles of the CTA.  The saved activation tile h is
// fetched by TMA INTO the staging buffer the result will leave from -- same 32 x 32 swizzled layout, so every lane
// replaces its own row in place -- and is requested one chunk ahead, as soon as the store that last read that buffer
// has let go of it.  State that lives across tiles is in `st`; a warp's chunks map onto st.acc[] as
// (column panel) * (chunks per half tile) + chunk, which the launcher keeps within four.
struct TcAuxState { uint32_t phase; float acc[4]; };
template <int SBUF>
__device__ __forceinline__ float* tc_stage_buf(float* stage, uint32_t count) { return stage + (SBUF == 2 ? (count & 1u) * (32 * 32) : 0); }
__device__ __forceinline__ void tc_aux_request(const CUtensorMap* tmap_aux, float* buf, uint64_t* aux_bar, int n0, long long m0) {
  mbar_expect_tx(aux_bar, 32 * 32 * 4);
  tma_load_3d(buf, tmap_aux, n0, (int)m0, 0, aux_bar);
}
template <int BN, int SBUF, int EPI_WARPS = 8>
__device__ __forceinline__ bool tc_epilogue_tile_aux(const TcArgs& g, const CUtensorMap* tmap_c, const CUtensorMap* tmap_aux, uint32_t t_base, int warp, int lane,
                                                     float* stage, uint64_t* aux_bar, volatile int* abort_flag, long long m_base, int nb,
                                                     bool next_valid, long long next_m_base, int next_nb, uint32_t& store_count, TcAuxState& st) {
  const int quad = warp & 3, half = (warp - 2) >> 2;
  const long long m0 = m_base + quad * 32;
  const uint32_t t_row = t_base + ((uint32_t)(quad * 32) << 16);
  const int rows_valid = (int)max(0LL, min((long long)32, (long long)g.M - m0));
  constexpr int HALF_COLS = BN / (EPI_WARPS / 4), CHUNKS = HALF_COLS / 32;
  static_assert(EPI_WARPS >= 8 && HALF_COLS >= 32, "a warp's share is whole 32-column chunks");
  if (next_valid && lane < CHUNKS && next_m_base + quad * 32 < g.M)   // the next tile's activation chunks: into L2 while this tile is worked on
    tma_prefetch_3d(tmap_aux, next_nb * BN + half * HALF_COLS + lane * 32, (int)(next_m_base + quad * 32), 0);
#pragma unroll 1
  for (int ci = 0; ci < CHUNKS; ++ci) {
    const int c0 = half * HALF_COLS + ci * 32;
    const int n0 = nb * BN + c0;
    float* buf = tc_stage_buf<SBUF>(stage, store_count);
    uint32_t r[32];
    tmem_ld32(t_row + (uint32_t)c0, r);
    tmem_ld_wait();
    if (!mbar_wait(aux_bar, st.phase, abort_flag)) return false;
    st.phase ^= 1;
    const bool row_ok = lane < rows_valid;                     // rows past M hold the map's fill value; they must not reach the sums
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float4* cell = (float4*)(buf + lane * 32 + ((c ^ (lane & 7)) << 2));
      const float4 a = *cell;
      const float x0 = __uint_as_float(r[4 * c]) * (1.f - a.x * a.x), x1 = __uint_as_float(r[4 * c + 1]) * (1.f - a.y * a.y);
      const float x2 = __uint_as_float(r[4 * c + 2]) * (1.f - a.z * a.z), x3 = __uint_as_float(r[4 * c + 3]) * (1.f - a.w * a.w);
      const float4 x = make_float4(row_ok ? x0 : 0.f, row_ok ? x1 : 0.f, row_ok ? x2 : 0.f, row_ok ? x3 : 0.f);
      *cell = x;
      r[4 * c] = __float_as_uint(x.x); r[4 * c + 1] = __float_as_uint(x.y); r[4 * c + 2] = __float_as_uint(x.z); r[4 * c + 3] = __float_as_uint(x.w);
    }
    fence_proxy_async();
    __syncwarp();
    ++store_count;
    if (lane == 0) {
      if (rows_valid > 0) tma_store_3d(tmap_c, buf, n0, (int)m0, 0);       // (a row block wholly past M is only padding)
      tma_store_commit();                                                  // one group per chunk, stored or not: the waits below count groups
      const bool more = ci + 1 < CHUNKS;
      if (more || next_valid) {
        tma_store_wait_read<SBUF - 1>();                                   // the store that last read the next chunk's buffer
        if (more) tc_aux_request(tmap_aux, tc_stage_buf<SBUF>(stage, store_count), aux_bar, n0 + 32, m0);
        else tc_aux_request(tmap_aux, tc_stage_buf<SBUF>(stage, store_count), aux_bar, next_nb * BN + half * HALF_COLS, next_m_base + quad * 32);
      }
    }
    {
      const float cs = tc_chunk_colsum(r, lane);               // lane l: the sum of the chunk's column l
      const int slot = (nb * CHUNKS + ci) & 3;
#pragma unroll
      for (int j = 0; j < 4; ++j) st.acc[j] += (j == slot) ? cs : 0.f;
    }
  }
  return true;
}

}  // namespace
