/*
 * CPU oracle for the Talos-XII dense neural path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C, f64 restatement of the reference crate's arithmetic (the crate is
 * Rust and cannot be built without a Rust toolchain).  Every function names the
 * reference file:line it follows.  Nothing in the shipped library links, loads
 * or calls this file; only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark do, and there only as the checker / the timed baseline.
 *
 * Parity status: the scalar primitives, matmul forward/backward, broadcast and
 * transpose are pinned by the reference's own known-answer tests (replayed in
 * the test-suite).  RMSNorm / RoPE / softmax / batched matmul / MLA / PPO-loss /
 * Adam VALUES are not fixed by any reference test ("parity unpinned"); they are
 * checked against central finite differences and cross-path consistency only.
 *
 * Build: gcc -O3 -mavx2 -mfma -fPIC -shared -pthread (see oracle/Makefile).
 * The explicit -mavx2 -mfma (rather than -march=native) keeps the binary
 * runnable on any x86-64 host with AVX2, like the crate's run-time dispatch
 * (src/simd.rs:8-17).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__AVX2__)
#include <immintrin.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Row-parallel helper standing in for Rayon's par_chunks_mut: the index range
 * [0,n) is cut into `threads` contiguous chunks, one OS thread each.          */
typedef void (*orc_range_fn)(long lo, long hi, void* arg);
typedef struct { orc_range_fn fn; long lo, hi; void* arg; } orc_job;
static void* orc_job_main(void* p) { orc_job* j = (orc_job*)p; j->fn(j->lo, j->hi, j->arg); return NULL; }

static void orc_parallel_for(long n, int threads, orc_range_fn fn, void* arg) {
  if (threads <= 1 || n < 2) { fn(0, n, arg); return; }
  if (threads > n) threads = (int)n;
  if (threads > 256) threads = 256;
  pthread_t tid[256]; orc_job job[256];
  long chunk = (n + threads - 1) / threads;
  int started = 0;
  for (int t = 0; t < threads; ++t) {
    long lo = t * chunk, hi = lo + chunk; if (hi > n) hi = n; if (lo >= hi) break;
    job[t].fn = fn; job[t].lo = lo; job[t].hi = hi; job[t].arg = arg;
    if (t == threads - 1 || hi == n) { fn(lo, hi, arg); break; }
    pthread_create(&tid[t], NULL, orc_job_main, &job[t]); ++started;
  }
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------------- */
/* src/simd.rs                                                                 */

/* add_scaled_row: out[i] += scale*row[i]  (src/simd.rs:2-31; AVX2+FMA body :149-188,
 * 8 doubles per iteration, then 4, then a scalar tail). */
ORC_API void orc_add_scaled_row(double* out, const double* row, double scale, long n) {
  long i = 0;
#if defined(__AVX2__) && defined(__FMA__)
  __m256d s = _mm256_set1_pd(scale);
  for (; i + 8 <= n; i += 8) {
    __m256d o0 = _mm256_loadu_pd(out + i), o1 = _mm256_loadu_pd(out + i + 4);
    o0 = _mm256_fmadd_pd(s, _mm256_loadu_pd(row + i), o0);
    o1 = _mm256_fmadd_pd(s, _mm256_loadu_pd(row + i + 4), o1);
    _mm256_storeu_pd(out + i, o0); _mm256_storeu_pd(out + i + 4, o1);
  }
  for (; i + 4 <= n; i += 4)
    _mm256_storeu_pd(out + i, _mm256_fmadd_pd(s, _mm256_loadu_pd(row + i), _mm256_loadu_pd(out + i)));
#endif
  for (; i < n; ++i) out[i] += scale * row[i];
}

/* dot_product: sum a[i]*b[i], two vector accumulators (src/simd.rs:34-63, :233-276). */
ORC_API double orc_dot_product(const double* a, const double* b, long n) {
  long i = 0; double sum = 0.0;
#if defined(__AVX2__) && defined(__FMA__)
  __m256d acc0 = _mm256_setzero_pd(), acc1 = _mm256_setzero_pd();
  for (; i + 8 <= n; i += 8) {
    acc0 = _mm256_fmadd_pd(_mm256_loadu_pd(a + i), _mm256_loadu_pd(b + i), acc0);
    acc1 = _mm256_fmadd_pd(_mm256_loadu_pd(a + i + 4), _mm256_loadu_pd(b + i + 4), acc1);
  }
  for (; i + 4 <= n; i += 4)
    acc0 = _mm256_fmadd_pd(_mm256_loadu_pd(a + i), _mm256_loadu_pd(b + i), acc0);
  double t[4]; _mm256_storeu_pd(t, _mm256_add_pd(acc0, acc1));
  sum = t[0] + t[1] + t[2] + t[3];
#endif
  for (; i < n; ++i) sum += a[i] * b[i];
  return sum;
}

/* vector_fma: dst[i] += a[i]*b[i]  (src/simd.rs:66-94). */
ORC_API void orc_vector_fma(double* dst, const double* a, const double* b, long n) {
  long i = 0;
#if defined(__AVX2__) && defined(__FMA__)
  for (; i + 4 <= n; i += 4)
    _mm256_storeu_pd(dst + i, _mm256_fmadd_pd(_mm256_loadu_pd(a + i), _mm256_loadu_pd(b + i), _mm256_loadu_pd(dst + i)));
#endif
  for (; i < n; ++i) dst[i] += a[i] * b[i];
}

/* vector_scale: row[i] *= scale  (src/simd.rs:362-401). */
ORC_API void orc_vector_scale(double* row, double scale, long n) {
  for (long i = 0; i < n; ++i) row[i] *= scale;
}

/* softmax_exp_sum: in-place exp(x - max); returns the sum; 0 for an empty row
 * (src/simd.rs:333-359). */
ORC_API double orc_softmax_exp_sum(double* row, long n) {
  if (n == 0) return 0.0;
  double mx = -INFINITY;
  for (long i = 0; i < n; ++i) if (row[i] > mx) mx = row[i];
  double sum = 0.0;
  for (long i = 0; i < n; ++i) { row[i] = exp(row[i] - mx); sum += row[i]; }
  return sum;
}

/* ------------------------------------------------------------------------- */
/* src/ppo.rs:24-106  advantage statistics                                     */
ORC_API double orc_sum_f64(const double* v, long n) { double s = 0; for (long i = 0; i < n; ++i) s += v[i]; return s; }
ORC_API double orc_sum_sq_diff(const double* v, double mean, long n) {
  double s = 0; for (long i = 0; i < n; ++i) { double d = v[i] - mean; s += d * d; } return s;
}
ORC_API void orc_normalize_slice(const double* v, double* out, double mean, double std, long n) {
  for (long i = 0; i < n; ++i) out[i] = (v[i] - mean) / std;
}

/* src/ppo.rs:444-480  RunningMeanStd: one-sample Welford-style update and the normalisation that uses it. */
ORC_API void orc_running_mean_std_update(double* count, double* mean, double* var, const double* x, long n) {
  for (long i = 0; i < n; ++i) {
    const double delta = x[i] - *mean, tot = *count + 1.0;
    const double new_mean = *mean + delta * 1.0 / tot;
    const double m2 = *var * *count + 0.0 * 1.0 + delta * delta * *count * 1.0 / tot;
    *mean = new_mean; *var = m2 / tot; *count = tot;
  }
}

/* src/ppo.rs:650-671  reward normalisation (clipped to +-10) and the reverse GAE scan over the whole rollout buffer:
 * delta = r_norm + gamma * V[t+1] * nonterminal - V[t];  gae = delta + gamma * lambda * nonterminal * gae_next;
 * V[len] = 0; advantages[t] = gae; returns[t] = gae + V[t]. */
ORC_API void orc_gae(const double* rewards, const double* values, const int32_t* terminals, long len, double gamma, double lambda,
                     double rew_mean, double rew_var, double* advantages, double* returns) {
  double last = 0.0;
  const double denom = sqrt(rew_var) + 1e-8;
  for (long t = len - 1; t >= 0; --t) {
    double r = (rewards[t] - rew_mean) / denom;
    if (r < -10.0) r = -10.0;
    if (r > 10.0) r = 10.0;
    const double nt = terminals[t] ? 0.0 : 1.0;
    const double v = values[t], vn = t < len - 1 ? values[t + 1] : 0.0;
    const double delta = r + gamma * vn * nt - v;
    const double gae = delta + gamma * lambda * nt * last;
    advantages[t] = gae; returns[t] = gae + v; last = gae;
  }
}

/* ------------------------------------------------------------------------- */
/* src/autograd.rs                                                             */

/* Tensor::rand LCG (src/autograd.rs:114-124): 31-bit value over a 32-bit divisor,
 * so r lies in [0, 0.5) -- reproduced on purpose. */
ORC_API void orc_lcg_rand(double* out, long n, double lo, double hi, uint64_t seed) {
  uint64_t x = seed;
  for (long i = 0; i < n; ++i) {
    x = x * 6364136223846793005ULL + 1ULL;
    double r = (double)(x >> 33) / 4294967295.0;
    out[i] = lo + r * (hi - lo);
  }
}

typedef struct { const double *A, *B, *G; double *C, *dA, *dB; long M, K, N; } orc_mm;

static void orc_mm_fwd_rows(long lo, long hi, void* p) {
  orc_mm* a = (orc_mm*)p; long K = a->K, N = a->N;
  for (long r = lo; r < hi; ++r) {
    double* out = a->C + r * N;
    for (long i = 0; i < K; ++i) {
      double s = a->A[r * K + i]; const double* brow = a->B + i * N;
      for (long c = 0; c < N; ++c) out[c] += s * brow[c];   /* plain mul+add loop, :246-248 */
    }
  }
}
/* Tensor::matmul forward (src/autograd.rs:200-258): C = A[M,K] . B[K,N]; output rows
 * in parallel once M*N*K >= 32768 (:222), i-k-j axpy order.  C is overwritten. */
ORC_API void orc_matmul_fwd(const double* A, const double* B, double* C, long M, long K, long N, int threads) {
  memset(C, 0, sizeof(double) * (size_t)(M * N));
  orc_mm a = {A, B, NULL, C, NULL, NULL, M, K, N};
  if (M * N * K < 32768) threads = 1;
  orc_parallel_for(M, threads, orc_mm_fwd_rows, &a);
}

static void orc_mm_bwd_lhs_rows(long lo, long hi, void* p) {
  orc_mm* a = (orc_mm*)p; long K = a->K, N = a->N;
  for (long r = lo; r < hi; ++r)
    for (long i = 0; i < K; ++i)
      a->dA[r * K + i] += orc_dot_product(a->G + r * N, a->B + i * N, N);
}
static void orc_mm_bwd_rhs_rows(long lo, long hi, void* p) {
  orc_mm* a = (orc_mm*)p; long K = a->K, N = a->N, M = a->M;
  for (long i = lo; i < hi; ++i) {
    double* row = a->dB + i * N;
    for (long r = 0; r < M; ++r) {
      double s = a->A[r * K + i];
      if (s == 0.0) continue;                               /* :340-342 */
      orc_add_scaled_row(row, a->G + r * N, s, N);
    }
  }
}
/* matmul backward (src/autograd.rs:268-351): dA += G.B^T via dot_product (:275-308),
 * dB += A^T.G via add_scaled_row (:310-350).  Either output may be NULL. */
ORC_API void orc_matmul_bwd(const double* A, const double* B, const double* G, double* dA, double* dB,
                            long M, long K, long N, int threads) {
  orc_mm a = {A, B, G, NULL, dA, dB, M, K, N};
  if (M * N * K < 32768) threads = 1;
  if (dA) orc_parallel_for(M, threads, orc_mm_bwd_lhs_rows, &a);
  if (dB) orc_parallel_for(K, threads, orc_mm_bwd_rhs_rows, &a);
}

/* broadcast_to_batch + Add (src/autograd.rs:511-547, :1608-1647; used by Linear::forward,
 * src/nn.rs:102-117): Y[r,:] += b. */
ORC_API void orc_bias_add(double* Y, const double* b, long M, long N) {
  for (long r = 0; r < M; ++r) for (long c = 0; c < N; ++c) Y[r * N + c] += b[c];
}
/* backward of broadcast_to_batch: db += column sums, serial over batch chunks (:539-543). */
ORC_API void orc_bias_bwd(const double* G, double* db, long M, long N) {
  for (long r = 0; r < M; ++r) for (long c = 0; c < N; ++c) db[c] += G[r * N + c];
}

/* Tensor::transpose (src/autograd.rs:632-739): generic N-d swap of two dims with a full
 * copy.  accumulate=0 is the forward (out[i] = in[old]), accumulate=1 the backward
 * scatter (in_grad[old] += g[i]) with `src` in the transposed layout. */
ORC_API void orc_transpose(const double* src, double* dst, const long* shape, int rank, int d0, int d1, int backward) {
  long nshape[8], st[8], nst[8], len = 1;
  for (int i = 0; i < rank; ++i) { nshape[i] = shape[i]; len *= shape[i]; }
  long t = nshape[d0]; nshape[d0] = nshape[d1]; nshape[d1] = t;
  st[rank - 1] = 1; nst[rank - 1] = 1;
  for (int i = rank - 2; i >= 0; --i) { st[i] = st[i + 1] * shape[i + 1]; nst[i] = nst[i + 1] * nshape[i + 1]; }
  for (long i = 0; i < len; ++i) {
    long tmp = i, c[8];
    for (int d = 0; d < rank; ++d) { c[d] = tmp / nst[d]; tmp %= nst[d]; }
    long s = c[d0]; c[d0] = c[d1]; c[d1] = s;
    long old = 0; for (int d = 0; d < rank; ++d) old += c[d] * st[d];
    if (backward) dst[old] += src[i]; else dst[i] = src[old];
  }
}

/* ------------------------------------------------------------------------- */
/* src/nn.rs                                                                   */

/* RMSNorm::forward (src/nn.rs:183-220): rms = sqrt(mean(x^2)+eps) (eps inside the sqrt),
 * xhat = x/rms, y = xhat*w; caches rms and xhat. */
ORC_API void orc_rmsnorm_fwd(const double* x, const double* w, double eps, long rows, long dim,
                             double* y, double* rms_cache, double* xhat) {
  for (long r = 0; r < rows; ++r) {
    const double* xr = x + r * dim; double ss = 0.0;
    for (long i = 0; i < dim; ++i) ss += xr[i] * xr[i];
    double rms = sqrt(ss / (double)dim + eps);
    rms_cache[r] = rms;
    for (long i = 0; i < dim; ++i) { double h = xr[i] / rms; xhat[r * dim + i] = h; y[r * dim + i] = h * w[i]; }
  }
}
/* RMSNorm backward (src/nn.rs:234-296): dx += (1/rms)(g*w - xhat*mean(g*w*xhat));
 * dw[i] += sum_rows g*xhat. */
ORC_API void orc_rmsnorm_bwd(const double* g, const double* w, const double* rms_cache, const double* xhat,
                             long rows, long dim, double* dx, double* dw) {
  for (long r = 0; r < rows; ++r) {
    double inv = 1.0 / rms_cache[r], dot = 0.0;
    for (long i = 0; i < dim; ++i) dot += g[r * dim + i] * w[i] * xhat[r * dim + i];
    double mean_dot = dot / (double)dim;
    for (long i = 0; i < dim; ++i)
      dx[r * dim + i] += inv * (g[r * dim + i] * w[i] - xhat[r * dim + i] * mean_dot);
  }
  if (dw) for (long i = 0; i < dim; ++i) {
    double s = 0.0; for (long r = 0; r < rows; ++r) s += g[r * dim + i] * xhat[r * dim + i];
    dw[i] += s;
  }
}

/* Linear::forward_inference (src/nn.rs:37-69): bias preload, axpy rows, skips zero inputs. */
ORC_API void orc_linear_forward_inference(const double* x, const double* W, const double* b, long rows,
                                          long in_dim, long out_dim, double* out) {
  for (long r = 0; r < rows; ++r) {
    double* o = out + r * out_dim;
    if (b) memcpy(o, b, sizeof(double) * (size_t)out_dim); else memset(o, 0, sizeof(double) * (size_t)out_dim);
    for (long i = 0; i < in_dim; ++i) {
      double s = x[r * in_dim + i]; if (s == 0.0) continue;
      orc_add_scaled_row(o, W + i * out_dim, s, out_dim);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* src/transformer.rs                                                          */

/* RoPE::precompute (src/transformer.rs:239-251): theta_i = 1/base^(2i/dim). */
ORC_API void orc_rope_table(long dim, long max_len, double base, double* cosv, double* sinv) {
  long h = dim / 2;
  for (long pos = 0; pos < max_len; ++pos)
    for (long i = 0; i < h; ++i) {
      double theta = 1.0 / pow(base, (double)(2 * i) / (double)dim);
      double ang = (double)pos * theta;
      cosv[pos * h + i] = cos(ang); sinv[pos * h + i] = sin(ang);
    }
}
/* RoPE::forward / backward (src/transformer.rs:253-337).  x is viewed as
 * [batches, seq_len, dim] where seq_len is the SECOND-TO-LAST axis of the caller's shape
 * (:262) -- for a [B,S,H,dr] input that axis is the head index, which is what the autograd
 * path rotates by.  backward=1 applies the transposed rotation and accumulates (:319-331). */
ORC_API void orc_rope(const double* x, double* out, const double* cosv, const double* sinv,
                      long batches, long seq_len, long dim, long start_pos, int backward) {
  long h = dim / 2;
  for (long b = 0; b < batches; ++b)
    for (long t = 0; t < seq_len; ++t) {
      long ci = (start_pos + t) * h, base = b * seq_len * dim + t * dim;
      for (long i = 0; i < h; ++i) {
        double c = cosv[ci + i], s = sinv[ci + i];
        double r1 = x[base + 2 * i], r2 = x[base + 2 * i + 1];
        if (!backward) { out[base + 2 * i] = r1 * c - r2 * s; out[base + 2 * i + 1] = r1 * s + r2 * c; }
        else { out[base + 2 * i] += r1 * c + r2 * s; out[base + 2 * i + 1] += -r1 * s + r2 * c; }
      }
    }
}
/* Token-position rotation of a [seq, heads*rope_dim] buffer as the graph-free paths do it
 * (src/transformer.rs:583-610 and :717-744): every head of token t is rotated by
 * start_pos + t; positions past the table are left unrotated (:586-588). */
ORC_API void orc_rope_token(const double* x, double* out, const double* cosv, const double* sinv, long table_len,
                            long batches, long seq_len, long heads, long rope_dim, long start_pos) {
  long h = rope_dim / 2;
  memcpy(out, x, sizeof(double) * (size_t)(batches * seq_len * heads * rope_dim));
  for (long b = 0; b < batches; ++b)
    for (long t = 0; t < seq_len; ++t) {
      long off = (start_pos + t) * h;
      if (off >= table_len) continue;
      for (long hd = 0; hd < heads; ++hd) {
        long base = ((b * seq_len + t) * heads + hd) * rope_dim;
        for (long i = 0; i < h; ++i) {
          double c = cosv[off + i], s = sinv[off + i];
          double r1 = x[base + 2 * i], r2 = x[base + 2 * i + 1];
          out[base + 2 * i] = r1 * c - r2 * s; out[base + 2 * i + 1] = r1 * s + r2 * c;
        }
      }
    }
}

typedef struct { const double *q, *k, *g; double *out, *dq, *dk; long seq, dim; } orc_bmm;

static void orc_qkt_fwd_b(long lo, long hi, void* p) {
  orc_bmm* a = (orc_bmm*)p; long S = a->seq, D = a->dim;
  for (long b = lo; b < hi; ++b)
    for (long i = 0; i < S; ++i) for (long j = 0; j < S; ++j)
      a->out[b * S * S + i * S + j] = orc_dot_product(a->q + b * S * D + i * D, a->k + b * S * D + j * D, D);
}
/* batched_matmul_qt_k forward (src/transformer.rs:877-909): out[b,i,j] = q[b,i,:].k[b,j,:]. */
ORC_API void orc_bmm_qkt_fwd(const double* q, const double* k, double* out, long B, long S, long D, int threads) {
  orc_bmm a = {q, k, NULL, out, NULL, NULL, S, D};
  orc_parallel_for(B, threads, orc_qkt_fwd_b, &a);
}
static void orc_qkt_bwd_b(long lo, long hi, void* p) {
  orc_bmm* a = (orc_bmm*)p; long S = a->seq, D = a->dim;
  for (long b = lo; b < hi; ++b) {
    const double *qs = a->q + b * S * D, *ks = a->k + b * S * D, *gs = a->g + b * S * S;
    double *dq = a->dq + b * S * D, *dk = a->dk + b * S * D;
    for (long i = 0; i < S; ++i) for (long j = 0; j < S; ++j) {
      double g = gs[i * S + j];
      for (long d = 0; d < D; ++d) { dq[i * D + d] += g * ks[j * D + d]; dk[j * D + d] += g * qs[i * D + d]; }
    }
  }
}
/* its backward (src/transformer.rs:920-955): scalar triple loop, accumulating. */
ORC_API void orc_bmm_qkt_bwd(const double* q, const double* k, const double* g, double* dq, double* dk,
                             long B, long S, long D, int threads) {
  orc_bmm a = {q, k, g, NULL, dq, dk, S, D};
  orc_parallel_for(B, threads, orc_qkt_bwd_b, &a);
}
static void orc_pv_fwd_b(long lo, long hi, void* p) {
  orc_bmm* a = (orc_bmm*)p; long S = a->seq, D = a->dim;   /* q = probs, k = v */
  for (long b = lo; b < hi; ++b)
    for (long i = 0; i < S; ++i) {
      double* o = a->out + b * S * D + i * D; memset(o, 0, sizeof(double) * (size_t)D);
      for (long j = 0; j < S; ++j) {
        double pv = a->q[b * S * S + i * S + j];
        if (fabs(pv) < 1e-9) continue;                      /* :989-991 */
        orc_add_scaled_row(o, a->k + b * S * D + j * D, pv, D);
      }
    }
}
/* batched_matmul_probs_v forward (src/transformer.rs:961-999), incl. the |p|<1e-9 skip. */
ORC_API void orc_bmm_pv_fwd(const double* probs, const double* v, double* out, long B, long S, long Dv, int threads) {
  orc_bmm a = {probs, v, NULL, out, NULL, NULL, S, Dv};
  orc_parallel_for(B, threads, orc_pv_fwd_b, &a);
}
static void orc_pv_bwd_b(long lo, long hi, void* p) {
  orc_bmm* a = (orc_bmm*)p; long S = a->seq, D = a->dim;
  for (long b = lo; b < hi; ++b) {
    const double *ps = a->q + b * S * S, *vs = a->k + b * S * D, *gs = a->g + b * S * D;
    double *dp = a->dq + b * S * S, *dv = a->dk + b * S * D;
    for (long i = 0; i < S; ++i) for (long d = 0; d < D; ++d) {
      double g = gs[i * D + d];
      for (long j = 0; j < S; ++j) { dp[i * S + j] += g * vs[j * D + d]; dv[j * D + d] += g * ps[i * S + j]; }
    }
  }
}
/* its backward (src/transformer.rs:1010-1046). */
ORC_API void orc_bmm_pv_bwd(const double* probs, const double* v, const double* g, double* dprobs, double* dv,
                            long B, long S, long Dv, int threads) {
  orc_bmm a = {probs, v, g, NULL, dprobs, dv, S, Dv};
  orc_parallel_for(B, threads, orc_pv_bwd_b, &a);
}

/* softmax over rows of length len (src/transformer.rs:1074-1087).  `causal_period` > 0 is an
 * extension the reference does not have: row r may only see columns j <= r % causal_period. */
ORC_API void orc_softmax_fwd(const double* x, double* y, long rows, long len, long causal_period) {
  for (long r = 0; r < rows; ++r) {
    long lim = causal_period > 0 ? (r % causal_period) + 1 : len;
    double mx = -INFINITY, sum = 0.0;
    for (long i = 0; i < lim; ++i) if (x[r * len + i] > mx) mx = x[r * len + i];
    for (long i = 0; i < lim; ++i) { double e = exp(x[r * len + i] - mx); y[r * len + i] = e; sum += e; }
    for (long i = 0; i < lim; ++i) y[r * len + i] /= sum;
    for (long i = lim; i < len; ++i) y[r * len + i] = 0.0;
  }
}
/* softmax backward (src/transformer.rs:1098-1117): dx_i += y_i (g_i - sum_j g_j y_j). */
ORC_API void orc_softmax_bwd(const double* y, const double* g, double* dx, long rows, long len) {
  for (long r = 0; r < rows; ++r) {
    double s = 0.0;
    for (long i = 0; i < len; ++i) s += g[r * len + i] * y[r * len + i];
    for (long i = 0; i < len; ++i) dx[r * len + i] += y[r * len + i] * (g[r * len + i] - s);
  }
}

/* ------------------------------------------------------------------------- */
/* src/rng.rs:14-103  SplitMix64-seeded xoshiro256**, 53-bit uniform, Box-Muller. */
typedef struct { uint64_t s[4]; } orc_rng;
static uint64_t orc_sm64(uint64_t* s) {
  *s += 0x9e3779b97f4a7c15ULL; uint64_t z = *s;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL; z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL; return z ^ (z >> 31);
}
static void orc_rng_seed(orc_rng* r, uint64_t seed) { for (int i = 0; i < 4; ++i) r->s[i] = orc_sm64(&seed); }
static inline uint64_t orc_rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
static uint64_t orc_rng_next(orc_rng* r) {
  uint64_t result = orc_rotl(r->s[1] * 5, 7) * 9, t = r->s[1] << 17;
  r->s[2] ^= r->s[0]; r->s[3] ^= r->s[1]; r->s[1] ^= r->s[2]; r->s[0] ^= r->s[3];
  r->s[2] ^= t; r->s[3] = orc_rotl(r->s[3], 45); return result;
}
static double orc_rng_f64(orc_rng* r) { return (double)(orc_rng_next(r) >> 11) * (1.0 / 9007199254740992.0); }

ORC_API void orc_rng_u64(uint64_t seed, uint64_t* out, long n) {
  orc_rng r; orc_rng_seed(&r, seed); for (long i = 0; i < n; ++i) out[i] = orc_rng_next(&r);
}
ORC_API void orc_rng_uniform(uint64_t seed, double lo, double hi, double* out, long n) {
  orc_rng r; orc_rng_seed(&r, seed); for (long i = 0; i < n; ++i) out[i] = lo + (hi - lo) * orc_rng_f64(&r);
}
/* next_f64_normal (src/rng.rs:84-103): z0 of Box-Muller only, u1 redrawn while 0. */
ORC_API void orc_rng_normal(uint64_t seed, double mean, double std, double* out, long n) {
  orc_rng r; orc_rng_seed(&r, seed);
  for (long i = 0; i < n; ++i) {
    double u1; do { u1 = orc_rng_f64(&r); } while (!(u1 > 0.0));
    double u2 = orc_rng_f64(&r);
    out[i] = mean + std * (sqrt(-2.0 * log(u1)) * cos(2.0 * M_PI * u2));
  }
}
/* next_u64_bounded (src/rng.rs:109-117): rejection sampling, no modulo bias. */
ORC_API void orc_rng_bounded(uint64_t seed, uint64_t range, int32_t* out, long n) {
  orc_rng r; orc_rng_seed(&r, seed);
  uint64_t threshold = (0ULL - range) % range;
  for (long i = 0; i < n; ++i) { uint64_t x; do { x = orc_rng_next(&r); } while (x < threshold); out[i] = (int32_t)(x % range); }
}
