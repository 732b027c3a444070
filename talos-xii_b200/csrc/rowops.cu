// Memory-bound row kernels: RMSNorm, softmax, RoPE.  One warp per row, 128-bit loads, the row
// held in registers between the reduction and the rescale, warp-shuffle reductions.
#include "common.cuh"

namespace {

constexpr int WARPS_PER_CTA = 8;
constexpr int MAX_VEC = 8;                 // 8 float4 per lane -> rows up to 1024 floats in registers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------- RMSNorm forward
// y = x * rsqrt(mean(x^2) + eps) * gamma; saves inv_rms per row.
template <int NVEC>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
rmsnorm_fwd_vec_kernel(const float4* __restrict__ x, const float4* __restrict__ gamma, float eps, long long rows,
                       int dim4, float* __restrict__ inv_rms, float4* __restrict__ y) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * WARPS_PER_CTA;
  float4 gam[NVEC];
#pragma unroll
  for (int v = 0; v < NVEC; ++v) { int c = lane + v * 32; gam[v] = c < dim4 ? __ldg(gamma + c) : make_float4(0, 0, 0, 0); }
  for (long long r = warp; r < rows; r += nwarps) {
    const float4* xr = x + r * dim4;
    float4 xv[NVEC]; float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NVEC; ++v) {
      int c = lane + v * 32;
      xv[v] = c < dim4 ? __ldcs(xr + c) : make_float4(0, 0, 0, 0);
      ss += xv[v].x * xv[v].x + xv[v].y * xv[v].y + xv[v].z * xv[v].z + xv[v].w * xv[v].w;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)(dim4 * 4) + eps);
    if (lane == 0 && inv_rms) inv_rms[r] = inv;
    float4* yr = y + r * dim4;
#pragma unroll
    for (int v = 0; v < NVEC; ++v) {
      int c = lane + v * 32;
      if (c < dim4) {
        float4 o; o.x = xv[v].x * inv * gam[v].x; o.y = xv[v].y * inv * gam[v].y;
        o.z = xv[v].z * inv * gam[v].z; o.w = xv[v].w * inv * gam[v].w;
        __stcs(yr + c, o);
      }
    }
  }
}

// Any dim / alignment: one warp per row, scalar strided loop, row re-read from cache.
__global__ void rmsnorm_fwd_generic_kernel(const float* __restrict__ x, const float* __restrict__ gamma, float eps,
                                           long long rows, int dim, float* __restrict__ inv_rms, float* __restrict__ y) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * WARPS_PER_CTA;
  for (long long r = warp; r < rows; r += nwarps) {
    const float* xr = x + r * dim; float ss = 0.f;
    for (int c = lane; c < dim; c += 32) ss += xr[c] * xr[c];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)dim + eps);
    if (lane == 0 && inv_rms) inv_rms[r] = inv;
    for (int c = lane; c < dim; c += 32) y[r * dim + c] = xr[c] * inv * gamma[c];
  }
}

// ---------------------------------------------------------------- RMSNorm backward
// dx (+)= inv*(dy*g - xhat*mean(dy*g*xhat)); per-CTA column partials of dy*xhat go to `partial`
// [gridDim.x][dim] and are summed in block order by colsum_partials_kernel (deterministic).
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
rmsnorm_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
                   const float* __restrict__ inv_rms, long long rows, int dim, float* __restrict__ dx, int acc_dx,
                   float* __restrict__ partial) {
  extern __shared__ float sh[];            // [WARPS_PER_CTA][dim] column partials
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  float* mine = sh + (size_t)w * dim;
  for (int c = lane; c < dim; c += 32) mine[c] = 0.f;
  const long long warp = (long long)blockIdx.x * WARPS_PER_CTA + w;
  const long long nwarps = (long long)gridDim.x * WARPS_PER_CTA;
  for (long long r = warp; r < rows; r += nwarps) {
    const float inv = inv_rms[r];
    const float* dyr = dy + r * dim; const float* xr = x + r * dim;
    float dot = 0.f;
    for (int c = lane; c < dim; c += 32) dot += dyr[c] * gamma[c] * (xr[c] * inv);
    dot = warp_sum(dot) / (float)dim;
    for (int c = lane; c < dim; c += 32) {
      float g = dyr[c], xh = xr[c] * inv;
      if (dx) { float v = inv * (g * gamma[c] - xh * dot); dx[r * dim + c] = acc_dx ? dx[r * dim + c] + v : v; }
      mine[c] += g * xh;
    }
  }
  __syncthreads();
  if (partial)
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      float s = 0.f;
      for (int i = 0; i < WARPS_PER_CTA; ++i) s += sh[(size_t)i * dim + c];
      partial[(size_t)blockIdx.x * dim + c] = s;
    }
}

// Vector variant (dim % 4 == 0, dim <= 1024, 16-byte aligned): the dy and x rows stay in registers between the
// reduction and the update, and each lane keeps its dgamma partials in registers across all the rows of its warp.
template <int NVEC>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
rmsnorm_bwd_vec_kernel(const float4* __restrict__ dy, const float4* __restrict__ x, const float4* __restrict__ gamma,
                       const float* __restrict__ inv_rms, long long rows, int dim4, float4* __restrict__ dx, int acc_dx,
                       float* __restrict__ partial) {
  extern __shared__ float sh[];            // [WARPS_PER_CTA][dim]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long warp = (long long)blockIdx.x * WARPS_PER_CTA + w;
  const long long nwarps = (long long)gridDim.x * WARPS_PER_CTA;
  float4 gam[NVEC], dg[NVEC];
#pragma unroll
  for (int v = 0; v < NVEC; ++v) { int c = lane + v * 32; gam[v] = c < dim4 ? __ldg(gamma + c) : make_float4(0, 0, 0, 0); dg[v] = make_float4(0, 0, 0, 0); }
  const float inv_dim = 1.f / (float)(dim4 * 4);
  for (long long r = warp; r < rows; r += nwarps) {
    const float inv = inv_rms[r];
    float4 g4[NVEC], x4[NVEC]; float dot = 0.f;
#pragma unroll
    for (int v = 0; v < NVEC; ++v) {
      int c = lane + v * 32;
      g4[v] = c < dim4 ? __ldcs(dy + r * dim4 + c) : make_float4(0, 0, 0, 0);
      x4[v] = c < dim4 ? __ldcs(x + r * dim4 + c) : make_float4(0, 0, 0, 0);
      x4[v].x *= inv; x4[v].y *= inv; x4[v].z *= inv; x4[v].w *= inv;               // x-hat
      dot += g4[v].x * gam[v].x * x4[v].x + g4[v].y * gam[v].y * x4[v].y + g4[v].z * gam[v].z * x4[v].z + g4[v].w * gam[v].w * x4[v].w;
    }
    dot = warp_sum(dot) * inv_dim;
#pragma unroll
    for (int v = 0; v < NVEC; ++v) {
      int c = lane + v * 32;
      if (c < dim4) {
        if (dx) {
          float4 o;
          o.x = inv * (g4[v].x * gam[v].x - x4[v].x * dot); o.y = inv * (g4[v].y * gam[v].y - x4[v].y * dot);
          o.z = inv * (g4[v].z * gam[v].z - x4[v].z * dot); o.w = inv * (g4[v].w * gam[v].w - x4[v].w * dot);
          if (acc_dx) { const float4 old = dx[r * dim4 + c]; o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
          __stcs(dx + r * dim4 + c, o);
        }
        dg[v].x += g4[v].x * x4[v].x; dg[v].y += g4[v].y * x4[v].y; dg[v].z += g4[v].z * x4[v].z; dg[v].w += g4[v].w * x4[v].w;
      }
    }
  }
  if (!partial) return;
#pragma unroll
  for (int v = 0; v < NVEC; ++v) { int c = lane + v * 32; if (c < dim4) ((float4*)(sh + (size_t)w * dim4 * 4))[c] = dg[v]; }
  __syncthreads();
  for (int c = threadIdx.x; c < dim4 * 4; c += blockDim.x) {
    float t = 0.f;
    for (int i = 0; i < WARPS_PER_CTA; ++i) t += sh[(size_t)i * dim4 * 4 + c];
    partial[(size_t)blockIdx.x * dim4 * 4 + c] = t;
  }
}

// Sums `nparts` partial rows of length `dim` in part order.  A CTA covers 32 columns x 8 part lanes;
// lane l sums parts l, l+8, ... then the eight lane sums are added in lane order (deterministic).
__global__ void __launch_bounds__(256)
colsum_partials_kernel(const float* __restrict__ partial, int nparts, int dim, float* __restrict__ out, int acc) {
  __shared__ float sh[8][33];
  const int cl = threadIdx.x & 31, pl = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float s = 0.f;
  if (c < dim) {
#pragma unroll 8
    for (int p = pl; p < nparts; p += 8) s += partial[(size_t)p * dim + c];
  }
  sh[pl][cl] = s;
  __syncthreads();
  if (pl == 0 && c < dim) {
    float t = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) t += sh[l][cl];
    out[c] = acc ? out[c] + t : t;
  }
}

// Column sums of a [rows, n] matrix, stage 1, any n: each CTA sums a contiguous slab of rows.
__global__ void colsum_stage1_kernel(const float* __restrict__ g, long long rows, int n, long long rows_per_cta,
                                     float* __restrict__ partial) {
  long long r0 = (long long)blockIdx.y * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  float s = 0.f;
#pragma unroll 8
  for (long long r = r0; r < r1; ++r) s += g[r * n + c];
  partial[(size_t)blockIdx.y * n + c] = s;
}

// Stage 1 for n % 4 == 0 and n <= 1024: 256 threads = (n/4 float4 columns) x (row lanes); every thread
// streams its rows with eight 128-bit loads in flight; row lanes are combined in lane order.
// DACT != 0 fuses the activation derivative of a Linear backward into the same pass: g_out = g * act'(saved)
// (g_out may be g) and the column sums are those of the product (dZ = dY * act'(.), db = colsum(dZ)).
template <int DACT>
__global__ void __launch_bounds__(256)
colsum_stage1_vec_kernel(const float4* g, float4* g_out, const float4* __restrict__ saved, long long rows, int n4, long long rows_per_cta,
                         float* __restrict__ partial) {
  extern __shared__ float4 shv[];                       // [row_lanes][n4]
  const int row_lanes = 256 / n4;
  const int cl = threadIdx.x % n4, rl = threadIdx.x / n4;
  const long long r0 = (long long)blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (rl < row_lanes) {
#pragma unroll 8
    for (long long r = r0 + rl; r < r1; r += row_lanes) {
      float4 v = __ldcs(g + r * n4 + cl);
      if (DACT) {
        const float4 a = __ldcs(saved + r * n4 + cl);
        v.x *= talos_dact(a.x, DACT); v.y *= talos_dact(a.y, DACT); v.z *= talos_dact(a.z, DACT); v.w *= talos_dact(a.w, DACT);
        g_out[r * n4 + cl] = v;
      }
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    shv[rl * n4 + cl] = s;
  }
  __syncthreads();
  if (rl == 0) {
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int l = 0; l < row_lanes; ++l) { const float4 v = shv[l * n4 + cl]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
    ((float4*)partial)[(size_t)blockIdx.x * n4 + cl] = t;
  }
}

// ---------------------------------------------------------------- softmax
// y = softmax(scale*x) over a row of `len` <= 32*NPL, one warp per row.
template <int NPL>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
softmax_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int len, float scale, int causal_period) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * WARPS_PER_CTA;
  for (long long r = warp; r < rows; r += nwarps) {
    const int lim = causal_period > 0 ? (int)(r % causal_period) + 1 : len;
    float v[NPL]; float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      int c = lane + i * 32;
      v[i] = c < lim ? __ldcs(x + r * len + c) * scale : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) { v[i] = (lane + i * 32) < lim ? expf(v[i] - mx) : 0.f; sum += v[i]; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < NPL; ++i) { int c = lane + i * 32; if (c < len) __stcs(y + r * len + c, v[i] * inv); }
  }
}

// Vector variant for row lengths 32*VEC*NV with 8*VEC-byte aligned rows: each lane owns NV chunks of VEC
// consecutive columns, so a warp moves 128*VEC bytes per load instruction.
template <int VEC> struct VecT;
template <> struct VecT<2> { using T = float2; };
template <> struct VecT<4> { using T = float4; };
template <int VEC> __device__ __forceinline__ void vec_to_arr(const typename VecT<VEC>::T& v, float* a);
template <> __device__ __forceinline__ void vec_to_arr<2>(const float2& v, float* a) { a[0] = v.x; a[1] = v.y; }
template <> __device__ __forceinline__ void vec_to_arr<4>(const float4& v, float* a) { a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; }
template <int VEC> __device__ __forceinline__ typename VecT<VEC>::T arr_to_vec(const float* a);
template <> __device__ __forceinline__ float2 arr_to_vec<2>(const float* a) { return make_float2(a[0], a[1]); }
template <> __device__ __forceinline__ float4 arr_to_vec<4>(const float* a) { return make_float4(a[0], a[1], a[2], a[3]); }

// Short rows: LPR lanes per row (a warp handles 32/LPR rows at once), NV float4 per lane, so the two
// reductions cost log2(LPR) shuffles for 32/LPR rows instead of 5 per row -- shuffle issue, not HBM, is what
// limits a one-row-per-warp softmax on 64-wide rows.
template <int LPR, int NV>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
softmax_fwd_vec_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, float scale, int causal_period) {
  constexpr int LEN = LPR * 4 * NV, RPW = 32 / LPR;
  const int lane = threadIdx.x & 31, sub = lane / LPR, l = lane % LPR;
  const long long warp = (long long)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * WARPS_PER_CTA;
  for (long long r0 = warp * RPW; r0 < rows; r0 += nwarps * RPW) {
    const long long r = r0 + sub;
    const bool ok = r < rows;
    const int lim = causal_period > 0 ? (int)(r % causal_period) + 1 : LEN;
    float4 v[NV]; float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      v[i] = ok ? __ldcs((const float4*)(x + r * LEN) + i * LPR + l) : make_float4(0.f, 0.f, 0.f, 0.f);
      const int c = (i * LPR + l) * 4;
      v[i].x = c + 0 < lim ? v[i].x * scale : -INFINITY; v[i].y = c + 1 < lim ? v[i].y * scale : -INFINITY;
      v[i].z = c + 2 < lim ? v[i].z * scale : -INFINITY; v[i].w = c + 3 < lim ? v[i].w * scale : -INFINITY;
      mx = fmaxf(fmaxf(mx, fmaxf(v[i].x, v[i].y)), fmaxf(v[i].z, v[i].w));
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * LPR + l) * 4;
      v[i].x = c + 0 < lim ? expf(v[i].x - mx) : 0.f; v[i].y = c + 1 < lim ? expf(v[i].y - mx) : 0.f;
      v[i].z = c + 2 < lim ? expf(v[i].z - mx) : 0.f; v[i].w = c + 3 < lim ? expf(v[i].w - mx) : 0.f;
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    if (ok) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        v[i].x *= inv; v[i].y *= inv; v[i].z *= inv; v[i].w *= inv;
        __stcs((float4*)(y + r * LEN) + i * LPR + l, v[i]);
      }
    }
  }
}

template <int NPL>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
softmax_bwd_kernel(const float* __restrict__ y, const float* dy, float* dx, long long rows,
                   int len, float scale, int acc) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * WARPS_PER_CTA;
  for (long long r = warp; r < rows; r += nwarps) {
    float yv[NPL], gv[NPL]; float s = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      int c = lane + i * 32;
      yv[i] = c < len ? __ldcs(y + r * len + c) : 0.f; gv[i] = c < len ? dy[r * len + c] : 0.f;   // dy may alias dx
      s += yv[i] * gv[i];
    }
    s = warp_sum(s);
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      int c = lane + i * 32;
      if (c < len) { float v = scale * yv[i] * (gv[i] - s); dx[r * len + c] = acc ? dx[r * len + c] + v : v; }
    }
  }
}

// ---------------------------------------------------------------- RoPE
// One thread per interleaved pair (2i, 2i+1) of a [outer, npos, inner, dim] tensor (any even dim).
__global__ void rope_kernel(const float2* __restrict__ x, float2* __restrict__ y, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long long table_len, long long total_pairs, int npos,
                            int inner, int half, long long start_pos, int inverse, int acc) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_pairs) return;
  int i = (int)(idx % half);
  long long rest = idx / half;               // (o*npos + p)*inner + in
  long long p = (rest / inner) % npos;
  long long toff = (start_pos + p) * half;
  float2 v = x[idx], o;
  if (toff >= table_len) { o = v; }
  else {
    float c = __ldg(cos_t + toff + i), s = __ldg(sin_t + toff + i);
    if (inverse) s = -s;
    o.x = v.x * c - v.y * s; o.y = v.x * s + v.y * c;
  }
  if (acc) { float2 old = y[idx]; o.x += old.x; o.y += old.y; }
  y[idx] = o;
}
// dim % 4 == 0, fewer than 2^31 pairs, 16-byte aligned buffers: one thread per TWO pairs (a 128-bit access),
// 32-bit index arithmetic, grid-stride loop.
__global__ void __launch_bounds__(256)
rope_vec_kernel(const float4* __restrict__ x, float4* __restrict__ y, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                unsigned table_len, unsigned total_quads, unsigned npos, unsigned inner, unsigned quads_per_row, unsigned start_pos,
                int inverse, int acc) {
  for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total_quads; idx += gridDim.x * blockDim.x) {
    const unsigned qi = idx % quads_per_row, rest = idx / quads_per_row;
    const unsigned p = (rest / inner) % npos;
    const unsigned toff = (start_pos + p) * (quads_per_row * 2);
    const float4 v = __ldcs(x + idx); float4 o;
    if (toff >= table_len) { o = v; }
    else {
      const float2 c = __ldg((const float2*)(cos_t + toff) + qi); float2 s = __ldg((const float2*)(sin_t + toff) + qi);
      if (inverse) { s.x = -s.x; s.y = -s.y; }
      o.x = v.x * c.x - v.y * s.x; o.y = v.x * s.x + v.y * c.x;
      o.z = v.z * c.y - v.w * s.y; o.w = v.z * s.y + v.w * c.y;
    }
    if (acc) { const float4 old = y[idx]; o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
    __stcs(y + idx, o);
  }
}

int row_grid(talos_ctx* ctx, int64_t rows) {
  int64_t want = ceil_div(rows, WARPS_PER_CTA);
  int64_t cap = (int64_t)ctx->sm_count * 8;          // 8 resident CTAs of 256 threads per SM
  return (int)std::max<int64_t>(1, std::min(want, cap));
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

TALOS_API talos_status talos_rmsnorm_fwd(talos_ctx* ctx, const float* x, const float* gamma, float eps, int64_t rows,
                                         int64_t dim, float* y, float* inv_rms) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && dim > 0 && dim < (1 << 24), TALOS_ERR_SHAPE, "RMSNorm dim mismatch");
  if (rows == 0) return TALOS_OK;
  TALOS_REQUIRE(x && gamma && y, TALOS_ERR_ARG, "null pointer");
  int grid = row_grid(ctx, rows);
  if (dim % 4 == 0 && dim <= 32 * 4 * MAX_VEC && aligned16(x) && aligned16(y) && aligned16(gamma)) {
    int dim4 = (int)(dim / 4), nvec = (int)ceil_div(dim4, 32);
    auto X = (const float4*)x; auto G = (const float4*)gamma; auto Y = (float4*)y;
#define TALOS_RMS_CASE(NV) case NV: rmsnorm_fwd_vec_kernel<NV><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(X, G, eps, rows, dim4, inv_rms, Y); break;
    switch (nvec) { TALOS_RMS_CASE(1) TALOS_RMS_CASE(2) TALOS_RMS_CASE(3) TALOS_RMS_CASE(4) TALOS_RMS_CASE(5) TALOS_RMS_CASE(6) TALOS_RMS_CASE(7) TALOS_RMS_CASE(8) }
#undef TALOS_RMS_CASE
  } else {
    rmsnorm_fwd_generic_kernel<<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(x, gamma, eps, rows, (int)dim, inv_rms, y);
  }
  talos_launched(ctx, "rmsnorm_fwd");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_rmsnorm_bwd(talos_ctx* ctx, const float* dy, const float* x, const float* gamma,
                                         const float* inv_rms, int64_t rows, int64_t dim, float* dx, float* dgamma,
                                         int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && dim > 0 && dim <= 1536, TALOS_ERR_SHAPE, "RMSNorm backward supports dim <= 1536");
  if (rows == 0) return TALOS_OK;
  TALOS_REQUIRE(dy && x && gamma && inv_rms, TALOS_ERR_ARG, "null pointer");
  int grid = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(rows, WARPS_PER_CTA), (int64_t)ctx->sm_count * 4));
  float* partial = dgamma ? (float*)talos_workspace(ctx, sizeof(float) * (size_t)grid * dim) : nullptr;
  size_t shmem = sizeof(float) * WARPS_PER_CTA * (size_t)dim;
  if (dim % 4 == 0 && dim <= 32 * 4 * MAX_VEC && aligned16(dy) && aligned16(x) && aligned16(gamma) && (!dx || aligned16(dx))) {
    const int dim4 = (int)(dim / 4), nvec = (int)ceil_div(dim4, 32);
    auto DY = (const float4*)dy; auto X = (const float4*)x; auto G = (const float4*)gamma; auto DX = (float4*)dx;
#define TALOS_RB_CASE(NV) case NV: rmsnorm_bwd_vec_kernel<NV><<<grid, WARPS_PER_CTA * 32, shmem, ctx->stream>>>(DY, X, G, inv_rms, rows, dim4, DX, accumulate & 1, partial); break;
    switch (nvec) { TALOS_RB_CASE(1) TALOS_RB_CASE(2) TALOS_RB_CASE(3) TALOS_RB_CASE(4) TALOS_RB_CASE(5) TALOS_RB_CASE(6) TALOS_RB_CASE(7) TALOS_RB_CASE(8) }
#undef TALOS_RB_CASE
  } else
  rmsnorm_bwd_kernel<<<grid, WARPS_PER_CTA * 32, shmem, ctx->stream>>>(dy, x, gamma, inv_rms, rows, (int)dim, dx,
                                                                        accumulate & 1, partial);
  talos_launched(ctx, "rmsnorm_bwd");
  if (dgamma) {
    colsum_partials_kernel<<<(unsigned)ceil_div(dim, 32), 256, 0, ctx->stream>>>(partial, grid, (int)dim, dgamma, (accumulate >> 1) & 1);
    talos_launched(ctx, "rmsnorm_dgamma");
  }
  TALOS_ENTRY_END
}

// out[c] (+)= sum_r g[r][c]; with dact != 0 the summand is g_out[r][c] = g[r][c] * act'(saved[r][c]), also written
// (vector path only: n % 4 == 0, n <= 1024, 16-byte aligned; returns false when the shape needs the plain path).
// `ext_partial` / `ext_cap` / `slabs_out`: leave the per-slab partial sums [slabs][n] in the caller's buffer and skip
// the second stage (the caller reduces them later); `out` is then unused.
static bool colsum_vec_launch(talos_ctx* ctx, const float* g, float* g_out, const float* saved, int dact, float* out, int64_t rows, int64_t n, int accumulate,
                              float* ext_partial = nullptr, int64_t ext_cap = 0, int* slabs_out = nullptr) {
  const bool vec = (n % 4 == 0) && n <= 1024 && aligned16(g) && (!dact || (aligned16(saved) && aligned16(g_out)));
  if (!vec) return false;
  const int n4 = (int)(n / 4);
  int64_t slabs = std::max<int64_t>(1, std::min<int64_t>(ceil_div(rows, 32), 4 * (int64_t)ctx->sm_count));
  int64_t rows_per = std::max<int64_t>(1, ceil_div(rows, slabs)); slabs = std::max<int64_t>(1, ceil_div(rows, rows_per));
  if (ext_partial && (ext_cap < slabs * n || !aligned16(ext_partial))) return false;
  float* partial = ext_partial ? ext_partial : (float*)talos_workspace(ctx, sizeof(float) * (size_t)slabs * n);
  size_t shmem = sizeof(float4) * (size_t)(256 / n4) * n4;
  auto G4 = (const float4*)g; auto O4 = (float4*)g_out; auto S4 = (const float4*)saved;
  switch (dact) {
    case 0: colsum_stage1_vec_kernel<0><<<(unsigned)slabs, 256, shmem, ctx->stream>>>(G4, O4, S4, rows, n4, rows_per, partial); break;
    case TALOS_ACT_RELU: colsum_stage1_vec_kernel<TALOS_ACT_RELU><<<(unsigned)slabs, 256, shmem, ctx->stream>>>(G4, O4, S4, rows, n4, rows_per, partial); break;
    case TALOS_ACT_TANH: colsum_stage1_vec_kernel<TALOS_ACT_TANH><<<(unsigned)slabs, 256, shmem, ctx->stream>>>(G4, O4, S4, rows, n4, rows_per, partial); break;
    case TALOS_ACT_SILU: colsum_stage1_vec_kernel<TALOS_ACT_SILU><<<(unsigned)slabs, 256, shmem, ctx->stream>>>(G4, O4, S4, rows, n4, rows_per, partial); break;
    default: throw talos_error(TALOS_ERR_ARG, "bad activation kind");
  }
  talos_launched(ctx, "colsum_stage1");
  if (ext_partial) { *slabs_out = (int)slabs; return true; }
  colsum_partials_kernel<<<(unsigned)ceil_div(n, 32), 256, 0, ctx->stream>>>(partial, (int)slabs, (int)n, out, accumulate ? 1 : 0);
  talos_launched(ctx, "colsum_stage2");
  return true;
}

// Internal (PPO trainer): the first stage only -- dZ = dY * act'(saved) when dact != 0 (dz may alias dy), per-slab
// column sums of dZ left in `partial` ([slabs][n]).  Returns the slab count, 0 when the shape is not served.
int talos_colsum_partials_launch(talos_ctx* ctx, const float* dy, float* dz, const float* saved, int dact, int64_t rows, int64_t n,
                                 float* partial, int64_t cap) {
  int slabs = 0;
  return colsum_vec_launch(ctx, dy, dz, saved, dact, nullptr, rows, n, 0, partial, cap, &slabs) ? slabs : 0;
}

// Internal (Linear backward, PPO trainer): dZ = dY * act'(saved) (dz may be dy), db (+)= colsum(dZ) in one pass.
bool talos_dact_colsum_launch(talos_ctx* ctx, const float* dy, float* dz, const float* saved, int dact, float* db, int64_t rows, int64_t n,
                              int accumulate) {
  return colsum_vec_launch(ctx, dy, dz, saved, dact, db, rows, n, accumulate);
}

TALOS_API talos_status talos_colsum(talos_ctx* ctx, const float* g, float* out, int64_t rows, int64_t n, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && n > 0 && n < (1 << 24), TALOS_ERR_SHAPE, "bad colsum shape");
  TALOS_REQUIRE(g && out, TALOS_ERR_ARG, "null pointer");
  if (colsum_vec_launch(ctx, g, nullptr, nullptr, 0, out, rows, n, accumulate)) return TALOS_OK;
  int64_t col_blocks = ceil_div(n, 128);
  int64_t slabs = std::max<int64_t>(1, std::min<int64_t>(ceil_div(rows, 64), (4 * (int64_t)ctx->sm_count) / col_blocks + 1));
  int64_t rows_per = std::max<int64_t>(1, ceil_div(rows, slabs)); slabs = std::max<int64_t>(1, ceil_div(rows, rows_per));
  float* partial = (float*)talos_workspace(ctx, sizeof(float) * (size_t)slabs * n);
  colsum_stage1_kernel<<<dim3((unsigned)col_blocks, (unsigned)slabs), 128, 0, ctx->stream>>>(g, rows, (int)n, rows_per, partial);
  talos_launched(ctx, "colsum_stage1");
  colsum_partials_kernel<<<(unsigned)ceil_div(n, 32), 256, 0, ctx->stream>>>(partial, (int)slabs, (int)n, out, accumulate ? 1 : 0);
  talos_launched(ctx, "colsum_stage2");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_softmax_fwd(talos_ctx* ctx, const float* x, float* y, int64_t rows, int64_t len, float scale,
                                         int64_t causal_period) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && len >= 0 && len <= 1024, TALOS_ERR_SHAPE, "softmax row length must be <= 1024");
  // a period longer than the row would let row r read columns of row r + 1 (and past the buffer on the last row)
  TALOS_REQUIRE(causal_period >= 0 && causal_period <= len, TALOS_ERR_SHAPE, "causal_period must be in [0, len]");
  if (rows == 0 || len == 0) return TALOS_OK;       // an empty row sums to 0 (src/simd.rs:335-337)
  TALOS_REQUIRE(x && y, TALOS_ERR_ARG, "null pointer");
  int grid = row_grid(ctx, len <= 128 ? ceil_div(rows, 4) : rows); int npl = (int)ceil_div(len, 32);
  if (aligned16(x) && aligned16(y) && (len == 64 || len == 128 || len == 256 || len == 512)) {
    const int cp = (int)causal_period;
    if (len == 64) softmax_fwd_vec_kernel<8, 2><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(x, y, rows, scale, cp);
    else if (len == 128) softmax_fwd_vec_kernel<8, 4><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(x, y, rows, scale, cp);
    else if (len == 256) softmax_fwd_vec_kernel<16, 4><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(x, y, rows, scale, cp);
    else softmax_fwd_vec_kernel<32, 4><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(x, y, rows, scale, cp);
    talos_launched(ctx, "softmax_fwd");
    return TALOS_OK;
  }
#define TALOS_SM_CASE(NP) if (npl <= NP) softmax_fwd_kernel<NP><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(x, y, rows, (int)len, scale, (int)causal_period); else
  TALOS_SM_CASE(1) TALOS_SM_CASE(2) TALOS_SM_CASE(4) TALOS_SM_CASE(8) TALOS_SM_CASE(16)
  softmax_fwd_kernel<32><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(x, y, rows, (int)len, scale, (int)causal_period);
#undef TALOS_SM_CASE
  talos_launched(ctx, "softmax_fwd");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_softmax_bwd(talos_ctx* ctx, const float* y, const float* dy, float* dx, int64_t rows,
                                         int64_t len, float scale, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(rows >= 0 && len >= 0 && len <= 1024, TALOS_ERR_SHAPE, "softmax row length must be <= 1024");
  if (rows == 0 || len == 0) return TALOS_OK;
  TALOS_REQUIRE(y && dy && dx, TALOS_ERR_ARG, "null pointer");
  int grid = row_grid(ctx, rows); int npl = (int)ceil_div(len, 32); int acc = accumulate ? 1 : 0;
#define TALOS_SM_CASE(NP) if (npl <= NP) softmax_bwd_kernel<NP><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(y, dy, dx, rows, (int)len, scale, acc); else
  TALOS_SM_CASE(1) TALOS_SM_CASE(2) TALOS_SM_CASE(4) TALOS_SM_CASE(8) TALOS_SM_CASE(16)
  softmax_bwd_kernel<32><<<grid, WARPS_PER_CTA * 32, 0, ctx->stream>>>(y, dy, dx, rows, (int)len, scale, acc);
#undef TALOS_SM_CASE
  talos_launched(ctx, "softmax_bwd");
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_rope_table(talos_ctx* ctx, int64_t dim, int64_t max_len, double base, float* cos_out,
                                        float* sin_out) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(dim > 0 && dim % 2 == 0 && max_len >= 0, TALOS_ERR_SHAPE, "RoPE dim must be even");
  TALOS_REQUIRE(cos_out && sin_out, TALOS_ERR_ARG, "null pointer");
  int64_t h = dim / 2; size_t n = (size_t)(max_len * h);
  std::string buf(sizeof(float) * 2 * n, '\0');
  float* hc = (float*)&buf[0]; float* hs = hc + n;
  for (int64_t pos = 0; pos < max_len; ++pos)
    for (int64_t i = 0; i < h; ++i) {
      double theta = 1.0 / pow(base, (double)(2 * i) / (double)dim), ang = (double)pos * theta;
      hc[pos * h + i] = (float)cos(ang); hs[pos * h + i] = (float)sin(ang);
    }
  TALOS_CHECK_CUDA(cudaMemcpyAsync(cos_out, hc, sizeof(float) * n, cudaMemcpyHostToDevice, ctx->stream));
  TALOS_CHECK_CUDA(cudaMemcpyAsync(sin_out, hs, sizeof(float) * n, cudaMemcpyHostToDevice, ctx->stream));
  TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));     // the staging buffer dies with this call
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_rope(talos_ctx* ctx, const float* x, float* y, const float* cos_t, const float* sin_t,
                                  int64_t table_len, int64_t outer, int64_t npos, int64_t inner, int64_t dim,
                                  int64_t start_pos, int32_t inverse, int32_t accumulate) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(dim > 0 && dim % 2 == 0 && outer >= 0 && npos >= 0 && inner >= 0 && start_pos >= 0, TALOS_ERR_SHAPE, "bad RoPE shape");
  int64_t pairs = outer * npos * inner * (dim / 2);
  if (pairs == 0) return TALOS_OK;
  TALOS_REQUIRE(x && y && cos_t && sin_t, TALOS_ERR_ARG, "null pointer");
  TALOS_REQUIRE(((uintptr_t)x & 7) == 0 && ((uintptr_t)y & 7) == 0, TALOS_ERR_ARG, "RoPE buffers must be 8-byte aligned");
  if (dim % 4 == 0 && pairs < (1LL << 31) && aligned16(x) && aligned16(y) && ((uintptr_t)cos_t % 8 == 0) && ((uintptr_t)sin_t % 8 == 0) &&
      table_len < (1LL << 31) && start_pos + npos < (1LL << 20)) {
    const unsigned quads = (unsigned)(pairs / 2);
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(quads, 256), (int64_t)ctx->sm_count * 16);
    rope_vec_kernel<<<grid, 256, 0, ctx->stream>>>((const float4*)x, (float4*)y, cos_t, sin_t, (unsigned)table_len, quads, (unsigned)npos,
                                                   (unsigned)inner, (unsigned)(dim / 4), (unsigned)start_pos, inverse ? 1 : 0, accumulate ? 1 : 0);
    talos_launched(ctx, "rope");
    return TALOS_OK;
  }
  rope_kernel<<<(unsigned)ceil_div(pairs, 256), 256, 0, ctx->stream>>>((const float2*)x, (float2*)y, cos_t, sin_t, table_len,
                                                                        pairs, (int)npos, (int)inner, (int)(dim / 2), start_pos,
                                                                        inverse ? 1 : 0, accumulate ? 1 : 0);
  talos_launched(ctx, "rope");
  TALOS_ENTRY_END
}
