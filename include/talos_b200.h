/*
 * talos_b200 -- C ABI of the B200 (sm_100a) implementation of the Talos-XII dense neural path.
 *
 * This is the surface a Rust `ffi.rs` (or any other FFI) binds.  Plain pointers and sizes only.
 * All matrices are fp32, row-major, in DEVICE memory unless a parameter name ends in `_host`.
 * Every function returns a talos_status (0 = OK), never throws across the boundary and never
 * aborts; talos_last_error_string() gives the message of the calling thread's last failure.
 * The reference crate reports the same conditions by panicking (assert!/assert_eq! on shapes,
 * src/autograd.rs:96-100, :201, :209, :1611; src/nn.rs:187); a host shim turns a non-zero status
 * back into a panic so GoodJobWorker::execute (src/worker.rs:110-132) still sees Err(String).
 *
 * Threading: a talos_ctx is one device + one stream; calls on one ctx must not overlap in time.
 * Work is enqueued on the ctx stream; only *_host entry points and talos_ctx_synchronize block.
 *
 * Each declaration cites the reference item it replaces (paths are relative to the reference
 * crate root).
 */
#ifndef TALOS_B200_H
#define TALOS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t talos_status;
enum {
  TALOS_OK = 0,
  TALOS_ERR_ARG = 1,      /* null pointer, bad enum, misaligned leading dimension */
  TALOS_ERR_SHAPE = 2,    /* the reference's "dimension mismatch" panics */
  TALOS_ERR_ALLOC = 3,
  TALOS_ERR_CUDA = 4,
  TALOS_ERR_NCCL = 5,
  TALOS_ERR_TIMEOUT = 6,  /* a bounded device-side wait gave up; the context stays usable */
  TALOS_ERR_UNSUPPORTED = 7
};

/* Arithmetic of the matrix products. */
enum {
  TALOS_MODE_FP32 = 0,    /* CUDA-core FFMA, fp32 exact products */
  TALOS_MODE_TF32X3 = 1,  /* tcgen05 tensor cores, 3 TF32 products per term: fp32-faithful (<=1e-5) */
  TALOS_MODE_TF32 = 2     /* tcgen05 tensor cores, single TF32 product: fast (<=2e-3) */
};
enum { TALOS_OP_N = 0, TALOS_OP_T = 1 };
enum { TALOS_ACT_NONE = 0, TALOS_ACT_RELU = 1, TALOS_ACT_TANH = 2, TALOS_ACT_SILU = 3 };
/* RoPE position convention. TOKEN: rotate by token position (src/transformer.rs:583-610).
 * HEAD_INDEX: the autograd path's behaviour, which rotates a [B,S,H,dr] tensor by the index
 * along its second-to-last axis, i.e. the head index (src/transformer.rs:262, :502-506). */
enum { TALOS_ROPE_TOKEN = 0, TALOS_ROPE_HEAD_INDEX = 1 };

typedef struct talos_ctx talos_ctx;

/* ---- context ------------------------------------------------------------------------------ */
/* `stream` is the cudaStream_t all work of this ctx is enqueued on (NULL: the default stream). */
talos_status talos_ctx_create(int32_t device, void* stream, talos_ctx** out);
talos_status talos_ctx_destroy(talos_ctx* ctx);
talos_status talos_ctx_synchronize(talos_ctx* ctx);
talos_status talos_ctx_set_stream(talos_ctx* ctx, void* stream);
/* Grow the ctx scratch buffer up front (split-K partials, dZ of Linear backward, attention
 * probabilities) so that later calls do not allocate. */
talos_status talos_ctx_reserve_workspace(talos_ctx* ctx, size_t bytes);
const char* talos_last_error_string(void);
/* 1 when the tcgen05 tensor-core GEMM passed its start-up self-check on this ctx and is in use
 * for TF32 / TF32X3 modes; 0 when those modes are being served by the fp32 CUDA-core kernel. */
int32_t talos_ctx_tensor_cores_active(talos_ctx* ctx);
/* The same as a three-way answer: 1 = self-check passed, tensor cores in use; 0 = no product large enough to need them
 * has run yet; -1 = the self-check FAILED and the fp32 kernel is standing in (results stay correct, speed does not). */
int32_t talos_ctx_tensor_cores_state(talos_ctx* ctx);
/* Number of kernels this library has launched on the ctx since creation. */
int64_t talos_ctx_launch_count(talos_ctx* ctx);
/* Test hook (no counterpart in the reference): writes `code` into the context's device-side error word from the
 * host, exactly where a kernel whose bounded wait gave up (1000..2999) or that met an out-of-range index (3000)
 * would write it.  The next entry point that blocks on the stream -- talos_ctx_synchronize, talos_copy_to_host,
 * talos_download_f64, talos_ppo_get_params_host, talos_ppo_last_loss, talos_ppo_update[_host] -- must then return
 * TALOS_ERR_TIMEOUT / TALOS_ERR_ARG and clear the word.  Lets the error path be tested without making a GPU misbehave. */
talos_status talos_debug_set_device_status(talos_ctx* ctx, int32_t code);
/* Test hook (no counterpart in the reference): makes a bounded wait inside the tensor-core GEMM kernel run out, the
 * way a lost copy would, WITHOUT faulting, trapping or hanging anything.  While skip_k_block >= 0, the first CTA of
 * every one-CTA tensor-core GEMM launched on this ctx leaves out the loads of that k-block (32 reduction elements) of
 * its first tile; the roles waiting for it poll `wait_spins` times (0 = the default 2^22, a few seconds; tests pass a
 * small value, >= 1024), give up, raise the device error word, let copies in flight land, free their tensor memory
 * and return.  The affected tile's results are undefined; the next blocking entry point returns TALOS_ERR_TIMEOUT.
 * skip_k_block = -1, wait_spins = 0 restores normal operation. */
talos_status talos_debug_gemm_stall(talos_ctx* ctx, int32_t skip_k_block, uint32_t wait_spins);

/* ---- device memory for hosts without a CUDA runtime binding of their own (the storage behind
 * Tensor.data / Tensor.grad, src/autograd.rs:15-20).  Copies are ordered on the ctx stream; the
 * *_host copies block until the host buffer may be reused / holds the data. */
/* talos_malloc / talos_free go through a per-context caching allocator (size classes: powers of two up to 1 MiB,
 * then multiples of 1 MiB): the reference allocates a fresh result and gradient buffer per op
 * (src/autograd.rs:94-107), so in steady state neither call reaches the CUDA driver or synchronises.  A freed block
 * is handed only to later work on the same ctx stream.  talos_free refuses a pointer it did not hand out. */
talos_status talos_malloc(talos_ctx* ctx, size_t bytes, void** out);
talos_status talos_free(talos_ctx* ctx, void* ptr);
/* Returns the allocator's idle blocks to the driver (waits for the stream first). */
talos_status talos_ctx_trim(talos_ctx* ctx);
/* stats4_host = {bytes handed out, bytes idle in the cache, cudaMalloc calls made, requests served from the cache}. */
talos_status talos_ctx_memory_stats(talos_ctx* ctx, int64_t* stats4_host);
/* Measurement aid, no counterpart in the reference: between _begin and _end every kernel launch made through this ctx is
 * followed by an event on its stream (at most 512).  _end waits for the stream and writes, for the first `capacity`
 * launches, the device time from the previous mark (the _begin call for the first) to the end of that launch in
 * microseconds and the launch's name (NUL-terminated, `name_stride` bytes apart); *count_out = launches recorded.
 * The events serialise nothing but cost about a microsecond each: not for timed regions. */
talos_status talos_ctx_timeline_begin(talos_ctx* ctx);
talos_status talos_ctx_timeline_end(talos_ctx* ctx, int32_t capacity, int32_t* count_out, float* us_out_host, char* names_out_host, int32_t name_stride);
talos_status talos_memset_zero(talos_ctx* ctx, void* ptr, size_t bytes);
talos_status talos_copy_from_host(talos_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
talos_status talos_copy_to_host(talos_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
talos_status talos_copy_device(talos_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes);
/* f64 host <-> fp32 device conversion at the Tensor boundary (the crate's Vec<f64>). */
talos_status talos_upload_f64(talos_ctx* ctx, float* dst_dev, const double* src_host, int64_t n);
talos_status talos_download_f64(talos_ctx* ctx, double* dst_host, const float* src_dev, int64_t n);

/* ---- GEMM: Tensor::matmul forward and both backward products ------------------------------ */
/* Optional fused epilogue, applied in this order to acc = op(A).op(B):
 *   v = acc + bias[n];  aux_out[m,n] = v;  v = act(v);  v *= dact(aux_in[m,n]);  C = v + beta*C.
 * dact is the activation derivative expressed on the saved tensor: RELU/TANH take the saved
 * OUTPUT y (y>0 ; 1-y^2), SILU takes the saved PRE-activation z. */
typedef struct talos_epilogue {
  const float* bias;      /* [N] or NULL: Linear's broadcast_to_batch + Add (src/nn.rs:102-117) */
  float* aux_out;         /* [M,N] pre-activation save or NULL */
  int64_t ld_aux_out;
  const float* aux_in;    /* [M,N] tensor the derivative is evaluated on, or NULL */
  int64_t ld_aux_in;
  int32_t act;            /* TALOS_ACT_* applied to the result */
  int32_t dact;           /* TALOS_ACT_* whose derivative multiplies the result */
  int32_t beta;           /* 0: overwrite C; 1: C += (the reference's `+=` gradient accumulation,
                             src/autograd.rs:304, :346) */
} talos_epilogue;

/* C[M,N] = op(A)[M,K] . op(B)[K,N].  op N: the operand is stored as written; op T: it is stored
 * transposed (A as [K,M], B as [N,K]).  Replaces Tensor::matmul forward (opA=N, opB=N;
 * src/autograd.rs:200-258), dLHS = G.B^T (opA=N, opB=T; :275-308) and dRHS = A^T.G
 * (opA=T, opB=N; :310-350). */
talos_status talos_gemm(talos_ctx* ctx, int32_t opA, int32_t opB, int64_t M, int64_t N, int64_t K,
                        const float* A, int64_t lda, const float* B, int64_t ldb, float* C, int64_t ldc,
                        int32_t mode, const talos_epilogue* epi);

/* `batch` independent products with element strides between consecutive matrices.  Replaces
 * batched_matmul_qt_k (opB=T; src/transformer.rs:877-958) and batched_matmul_probs_v
 * (src/transformer.rs:961-1050) and their backward products. */
talos_status talos_gemm_batched(talos_ctx* ctx, int32_t opA, int32_t opB, int64_t M, int64_t N, int64_t K,
                                const float* A, int64_t lda, int64_t strideA, const float* B, int64_t ldb,
                                int64_t strideB, float* C, int64_t ldc, int64_t strideC, int64_t batch,
                                int32_t beta, int32_t mode);

/* ---- Linear (src/nn.rs:12-142), weight [in,out] row-major, y = act(x.W + b) ---------------- */
/* z_save (nullable) receives the pre-activation (needed by SILU backward). */
talos_status talos_linear_fwd(talos_ctx* ctx, const float* x, const float* W, const float* bias, float* y,
                              float* z_save, int64_t rows, int64_t in_features, int64_t out_features,
                              int32_t act, int32_t mode);
/* saved = y for RELU/TANH/NONE, z for SILU.  dx/dW/db may each be NULL.  accumulate bit0: dx +=,
 * bit1: dW +=, bit2: db += (the reference always accumulates; fresh buffers pass 0). */
talos_status talos_linear_bwd(talos_ctx* ctx, const float* x, const float* W, const float* saved,
                              const float* dy, float* dx, float* dW, float* db, int64_t rows,
                              int64_t in_features, int64_t out_features, int32_t act, int32_t mode,
                              int32_t accumulate);
/* broadcast_to_batch + Add and its backward column sum (src/autograd.rs:511-547). */
talos_status talos_bias_add(talos_ctx* ctx, float* y, const float* bias, int64_t rows, int64_t n);
talos_status talos_colsum(talos_ctx* ctx, const float* g, float* out, int64_t rows, int64_t n, int32_t accumulate);
/* Same result as talos_colsum for callers that must not allocate (no counterpart in the reference, which
 * has no device memory to manage).  talos_colsum takes its partial-sum scratch from the context and may
 * grow it with cudaMalloc, which synchronises the whole device: a trainer thread doing that stalls every
 * other thread's kernels, and a host that gave all device memory to its own pool has none left to hand out.
 * This variant keeps the scratch in a fixed 2 MiB array inside the library image and never allocates or
 * frees anything.  Each GPU on which a context has been created (or this function called) holds the array
 * until the process exits: talos_ctx_create looks up the array's device address, which is the moment the
 * driver loads the module and sets the 2 MiB aside -- so create the context at start-up, before the
 * allocation-free phase of the caller begins and before any stream capture.  If that look-up failed, the
 * first call repeats it (and may then allocate, once).
 * Limits: n <= 1024 columns; wider input is refused with TALOS_ERR_UNSUPPORTED.
 * All calls share the one array: two calls whose kernels overlap on the GPU (different streams or
 * contexts) race on it, so keep them on one stream or serialise them.  Nothing in the array has to be
 * cleared between calls: each call overwrites every element it later reads. */
talos_status talos_colsum_noalloc(talos_ctx* ctx, const float* g, float* out, int64_t rows, int64_t n, int32_t accumulate);

/* ---- the slice primitives of src/simd.rs on device vectors ----------------------------------- */
/* add_scaled_row (src/simd.rs:2-32): out[i] += scale * row[i]. */
talos_status talos_axpy(talos_ctx* ctx, float* out, const float* row, float scale, int64_t n);
/* dot_product (src/simd.rs:34-63): out[0] (+)= sum_i a[i] * b[i]; out is a device scalar. */
talos_status talos_dot(talos_ctx* ctx, const float* a, const float* b, int64_t n, float* out, int32_t accumulate);
/* vector_fma (src/simd.rs:66-94): dst[i] += a[i] * b[i]. */
talos_status talos_vector_fma(talos_ctx* ctx, float* dst, const float* a, const float* b, int64_t n);
/* vector_scale (src/simd.rs:362-379): row[i] *= scale. */
talos_status talos_vector_scale(talos_ctx* ctx, float* row, float scale, int64_t n);
/* softmax_exp_sum (src/simd.rs:333-359): row[i] = exp(row[i] - max(row)) in place, sum_out[0] (device) = their sum;
 * an empty row gives 0. */
talos_status talos_softmax_exp_sum(talos_ctx* ctx, float* row, int64_t n, float* sum_out);

/* ---- RMSNorm (src/nn.rs:145-304): rms = sqrt(mean(x^2)+eps), y = x/rms*gamma --------------- */
/* inv_rms [rows] is the only thing saved for backward (x-hat is recomputed). */
talos_status talos_rmsnorm_fwd(talos_ctx* ctx, const float* x, const float* gamma, float eps, int64_t rows,
                               int64_t dim, float* y, float* inv_rms);
/* accumulate bit0: dx +=, bit1: dgamma +=. */
talos_status talos_rmsnorm_bwd(talos_ctx* ctx, const float* dy, const float* x, const float* gamma,
                               const float* inv_rms, int64_t rows, int64_t dim, float* dx, float* dgamma,
                               int32_t accumulate);

/* ---- RoPE (src/transformer.rs:220-371) ---------------------------------------------------- */
/* cos/sin tables [max_len, dim/2] computed in f64 on the host as RoPE::precompute does
 * (src/transformer.rs:239-251), rounded to fp32, written to device memory. */
talos_status talos_rope_table(talos_ctx* ctx, int64_t dim, int64_t max_len, double base, float* cos_out,
                              float* sin_out);
/* x viewed as [outer, npos, inner, dim]; element (o,p,i,:) is rotated by position start_pos+p
 * over interleaved pairs (2i,2i+1).  TOKEN on [B,S,H,dr]: outer=B,npos=S,inner=H.  HEAD_INDEX
 * (RoPE::forward as the autograd path calls it): outer=B*S,npos=H,inner=1.  inverse=1 applies the
 * transposed rotation (the backward, :319-331); accumulate=1 adds into y.  Positions at or past
 * table_len are copied unrotated (src/transformer.rs:351, :586-588). */
talos_status talos_rope(talos_ctx* ctx, const float* x, float* y, const float* cos_t, const float* sin_t,
                        int64_t table_len, int64_t outer, int64_t npos, int64_t inner, int64_t dim,
                        int64_t start_pos, int32_t inverse, int32_t accumulate);

/* ---- softmax (src/transformer.rs:1052-1121; src/simd.rs:333-359) -------------------------- */
/* y = softmax(scale * x) over rows of length len.  causal_period > 0 (not in the reference):
 * row r sees columns j <= r % causal_period; 0 <= causal_period <= len, anything else is TALOS_ERR_SHAPE. */
talos_status talos_softmax_fwd(talos_ctx* ctx, const float* x, float* y, int64_t rows, int64_t len, float scale,
                               int64_t causal_period);
/* dx (+)= scale * y * (dy - sum_j dy_j y_j). */
talos_status talos_softmax_bwd(talos_ctx* ctx, const float* y, const float* dy, float* dx, int64_t rows,
                               int64_t len, float scale, int32_t accumulate);

/* ---- attention core: scores -> scale -> softmax -> .V ---------------------------------------- */
/* q,k [BH,S,dqk], v [BH,S,dv], out [BH,S,dv]; probs (nullable) [BH,S,S] is written when the tape
 * needs it.  Replaces batched_matmul_qt_k + scale_tensor + softmax + batched_matmul_probs_v
 * (src/transformer.rs:539-550).  mode FP32: one fused CUDA-core kernel, scores never leave the SM,
 * S <= 128.  mode TF32 / TF32X3: two batched tensor-core GEMMs around an in-place softmax (S <= 1024);
 * shapes the tensor-core GEMM does not take fall back to the fused kernel. */
talos_status talos_attention_fwd(talos_ctx* ctx, const float* q, const float* k, const float* v, float* out,
                                 float* probs, int64_t BH, int64_t S, int64_t dqk, int64_t dv, float scale,
                                 int32_t causal, int32_t mode);
/* Backward from saved probs (the closures at src/transformer.rs:920-955, :1010-1046, :1063-1068,
 * :1098-1117): dq,dk,dv are overwritten.  The four products run as batched GEMMs in `mode`. */
talos_status talos_attention_bwd(talos_ctx* ctx, const float* q, const float* k, const float* v,
                                 const float* probs, const float* dout, float* dq, float* dk, float* dv,
                                 int64_t BH, int64_t S, int64_t dqk, int64_t dvdim, float scale, int32_t mode);

/* ---- advantage estimation (src/ppo.rs:650-675) --------------------------------------------- */
/* Reward normalisation with the running statistics (RunningMeanStd::normalize, src/ppo.rs:476-478:
 * (r - mean) / (sqrt(var) + 1e-8)), clipped to +-10 (:655), then the reverse GAE scan over the whole
 * rollout buffer (:658-671): delta = r + gamma * V[t+1] * nonterminal - V[t] with V[len] = 0,
 * gae = delta + gamma * lambda * nonterminal * gae_next; advantages[t] = gae, returns[t] = gae + V[t].
 * terminals: int32, non-zero where is_terminals[t].  The crate's constants are gamma 0.99,
 * lambda 0.95 (:18-19).  All arrays on the device, length len. */
talos_status talos_gae(talos_ctx* ctx, const float* rewards, const float* values, const int32_t* terminals, int64_t len,
                       float gamma, float lambda, float rew_mean, float rew_var, float* advantages, float* returns);
/* Advantage normalisation (src/ppo.rs:673-675, sum_f64 / sum_sq_diff / normalize_slice at :24-244):
 * y = (x - mean) / (sqrt(sum((x - mean)^2) / n) + 1e-8).  stats (nullable, device, 2 floats) receives
 * the mean and that denominator.  y may alias x. */
talos_status talos_normalize_slice(talos_ctx* ctx, const float* x, int64_t n, float* y, float* stats);

/* ---- dueling double-DQN train step (src/dqn.rs) --------------------------------------------- */
/* DuelingQNetwork::forward_impl, batch branch (src/dqn.rs:76-93): q = v + adv - mean_a(adv), which the
 * crate spells as three matmuls with constant ones matrices.  v [B,1], adv [B,A], q [B,A]. */
talos_status talos_dueling_combine_fwd(talos_ctx* ctx, const float* v, const float* adv, float* q, int64_t B, int64_t A);
/* Its backward: dv[b] (+)= sum_a dq[b,a]; dadv[b,a] (+)= dq[b,a] - mean_a dq[b,:].  dv or dadv may be null. */
talos_status talos_dueling_combine_bwd(talos_ctx* ctx, const float* dq, float* dv, float* dadv, int64_t B, int64_t A, int32_t accumulate);
/* Double-DQN targets (src/dqn.rs:524-556): target[b] = r[b] + gamma * q_next_target[b, argmax_a q_next_eval[b,a]] * (1 - done[b]);
 * the first maximum wins (strict >, as the crate's loop).  dones holds 0.0 / 1.0. */
talos_status talos_dqn_target(talos_ctx* ctx, const float* q_next_eval, const float* q_next_target, const float* rewards,
                              const float* dones, float gamma, float* target, int64_t B, int64_t A);
/* q_sel[b] = q[b, actions[b]] (the mask product + matmul with ones, src/dqn.rs:516-520); loss[0] = mean_b (q_sel - target)^2
 * (mse_loss, src/autograd.rs:1599-1603); dq (nullable) [B,A] is OVERWRITTEN with dloss/dq. */
talos_status talos_dqn_loss_fwd_bwd(talos_ctx* ctx, const float* q, const int32_t* actions, const float* target, float* loss,
                                    float* dq, int64_t B, int64_t A);
/* DuelingQNetwork::soft_update (src/dqn.rs:129-150): target = target * (1 - tau) + source * tau over n parameters. */
talos_status talos_soft_update(talos_ctx* ctx, float* target_params, const float* source_params, float tau, int64_t n);

/* ---- batched rollout inference ------------------------------------------------------------ */
/* One decode step of MultiHeadLatentAttention::forward_inference_cached (src/transformer.rs:688-841)
 * for N independent simulations at once -- the attention part of ActorCritic::step_inference_cached
 * (src/ppo.rs:391-432) as the simulator calls it once per pull (src/sim.rs:208), followed by the
 * sliding-window prune (src/transformer.rs:843-874, src/sim.rs:171-175, :578).
 *   q_c, k_c, v_c [N, H*dh], q_r, k_r [N, H*dr]: the five projections of the new token (Linear outputs);
 *   pos [N] (device): each simulation's absolute token position (the `start_pos` argument);
 *   k_cache [N,H,cap,dh+dr], v_cache [N,H,cap,dh]: per-simulation rings, cap = context_len + 1;
 *   out [N, H*dh]: attention output, ready for w_o.
 * Rotates q_r and k_r by pos (interleaved pairs, positions past the table unrotated), writes
 * k = [k_c | rot(k_r)] and v_c into ring slot pos % cap, attends over the min(pos+1, cap) live slots
 * with `scale`.  Does not change pos: call talos_decode_advance after the step. */
talos_status talos_mla_decode_step(talos_ctx* ctx, const float* q_c, const float* q_r, const float* k_c, const float* k_r,
                                   const float* v_c, const float* cos_t, const float* sin_t, int64_t table_len,
                                   const int32_t* pos, float* k_cache, float* v_cache, float* out, int64_t N, int64_t H,
                                   int64_t dh, int64_t dr, int64_t cap, float scale);
/* pos[n] = reset[n] ? 0 : pos[n] + 1.  reset (nullable, device): simulations that start a new episode,
 * i.e. whose KVCache the simulator clears (src/transformer.rs:420-424). */
talos_status talos_decode_advance(talos_ctx* ctx, int32_t* pos, const int32_t* reset, int64_t N);

/* ---- layout ops --------------------------------------------------------------------------- */
/* Tensor::transpose (src/autograd.rs:632-739): swap two axes of a rank<=6 tensor (full copy).
 * accumulate=1 adds into y (its backward). `shape` is the INPUT shape, host memory. */
talos_status talos_transpose(talos_ctx* ctx, const float* x, float* y, const int64_t* shape_host, int32_t rank,
                             int32_t dim0, int32_t dim1, int32_t accumulate);
/* concat_last_dim (src/transformer.rs:1123-1183) and its backward split. */
talos_status talos_concat_last(talos_ctx* ctx, const float* a, const float* b, float* out, int64_t rows,
                               int64_t da, int64_t db);
talos_status talos_split_last(talos_ctx* ctx, const float* g, float* ga, float* gb, int64_t rows, int64_t da,
                              int64_t db, int32_t accumulate);
/* LuckTransformer::last_token (src/transformer.rs:92-109): [B,S,D] -> [B,D]. */
talos_status talos_last_token(talos_ctx* ctx, const float* x, float* y, int64_t B, int64_t S, int64_t D);

/* ---- elementwise + reductions (src/autograd.rs:356-509, :741-768, :1608-1862) ------------- */
enum {
  TALOS_EW_RELU = 1, TALOS_EW_TANH = 2, TALOS_EW_SILU = 3, TALOS_EW_EXP = 4, TALOS_EW_LOG = 5, TALOS_EW_SIN = 6,
  TALOS_EW_COS = 7, TALOS_EW_SQRT = 8, TALOS_EW_CLIP = 9, TALOS_EW_NEG = 10, TALOS_EW_SCALE = 11,
  TALOS_EW_ADD = 20, TALOS_EW_SUB = 21, TALOS_EW_MUL = 22, TALOS_EW_DIV = 23
};
/* y = f(x; p0, p1) (CLIP: min,max; SCALE: factor). */
talos_status talos_eltwise_unary(talos_ctx* ctx, int32_t op, const float* x, float* y, int64_t n, float p0, float p1);
/* dx += dy * f'(x)   (always accumulates, like the reference's closures). */
talos_status talos_eltwise_unary_bwd(talos_ctx* ctx, int32_t op, const float* x, const float* dy, float* dx,
                                     int64_t n, float p0, float p1);
talos_status talos_eltwise_binary(talos_ctx* ctx, int32_t op, const float* a, const float* b, float* y, int64_t n);
/* da += ..., db += ... for ADD/SUB/MUL/DIV; a and b (and da, db) may alias (x*x), which the
 * reference special-cases at src/autograd.rs:1729, :1792. */
talos_status talos_eltwise_binary_bwd(talos_ctx* ctx, int32_t op, const float* a, const float* b, const float* dy,
                                      float* da, float* db, int64_t n);
/* out[0] (+)= scale * sum(x): Tensor::sum / mean forward, broadcast backward. */
talos_status talos_reduce_sum(talos_ctx* ctx, const float* x, int64_t n, float scale, float* out, int32_t accumulate);
/* y[i] (+)= scale * s[0]: Tensor::broadcast forward, sum / mean backward. */
talos_status talos_fill_from_scalar(talos_ctx* ctx, const float* s, float scale, float* y, int64_t n, int32_t accumulate);

/* ---- PPO loss and Adam (src/ppo.rs) ------------------------------------------------------- */
/* One pass over a minibatch of the per-sample loss of PPO::update (src/ppo.rs:702-755):
 * log-softmax, ratio, clipped surrogate (surr1 iff surr1 < surr2), (v-R)^2, entropy; writes
 * dL/dlogits [n,A] (row stride ld_out) and dL/dvalue, both already divided by `denom`, and ADDS
 * {sum loss, sum kl, n} to stats[0..2].  values/dvalues have element stride `value_stride`. */
talos_status talos_ppo_loss_fwd_bwd(talos_ctx* ctx, const float* logits, int64_t ld_logits, const float* values,
                                    int64_t value_stride, const int32_t* actions, const float* old_logp,
                                    const float* adv, const float* ret, int64_t n, int32_t n_actions, float clip,
                                    float c_value, float c_entropy, float denom, float* dlogits, int64_t ld_out,
                                    float* dvalues, int64_t dvalue_stride, float* stats);
/* Adam::step over a flat buffer (src/ppo.rs:519-533): g is first multiplied by grad_scale;
 * clip_norm > 0 adds the DQN optimizer's global-norm clip (src/dqn.rs:209-222). t is the step
 * number after the increment (>= 1). */
talos_status talos_adam_step(talos_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n,
                             int64_t t, float lr, float beta1, float beta2, float eps, float grad_scale,
                             float clip_norm);

/* The DQN optimizer's step on ONE tensor of a model whose global gradient norm spans several tensors
 * (src/dqn.rs:209-222 sums g^2 over ALL parameters first): sumsq_dev[0] (device) holds that sum -- e.g. accumulated
 * with talos_dot(g, g, n, sumsq, 1) per tensor -- and the step scales g by clip_norm / sqrt(sum) when the norm exceeds
 * clip_norm.  Nothing comes back to the host. */
talos_status talos_adam_step_global_clip(talos_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n,
                                         int64_t t, float lr, float beta1, float beta2, float eps, float grad_scale,
                                         const float* sumsq_dev, float clip_norm);

/* ---- seeded synthetic inputs: src/rng.rs:14-117 (SplitMix64 -> xoshiro256**) on the host ---- */
talos_status talos_rng_uniform_host(uint64_t seed, float lo, float hi, float* out_host, int64_t n);
talos_status talos_rng_normal_host(uint64_t seed, float mean, float std, float* out_host, int64_t n);
talos_status talos_rng_bounded_host(uint64_t seed, uint32_t range, int32_t* out_host, int64_t n);
/* Tensor::rand's LCG (src/autograd.rs:114-124), used by Linear::new (src/nn.rs:22-23). */
talos_status talos_lcg_rand_host(uint64_t seed, double lo, double hi, double* out_host, int64_t n);

#ifdef __cplusplus
}
#endif
#endif /* TALOS_B200_H */
