// Data-parallel PPO actor-critic update: the optimisation loops of PPO::update (src/ppo.rs:680-769)
// for an MLP actor-critic, one fused sequence of GEMM / loss / Adam launches per minibatch.
#include <functional>
#include <vector>

#include "comm.cuh"

// internal launchers of other translation units
void talos_adam_launch(talos_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, int64_t t, float lr, float b1,
                       float b2, float eps, float grad_scale, const float* count_ptr, float clip_norm, float* stats_out);

struct talos_ppo {
  talos_ctx* ctx; talos_ppo_config cfg;
  int HP;                              // padded width of the fused head [policy | value | 0...]
  int64_t n_int;                       // floats of the internal flat layout
  int64_t o_w1, o_b1, o_w2, o_b2, o_wh, o_bh;
  float *params, *grads, *m, *v;       // grads has 4 extra floats: {sum loss, sum kl, count, unused}
  float *h1, *h2, *z, *dz, *dh2, *dh1; // activations for one minibatch
  float* step_stats;                   // [max_steps][4] copy of the tail after each step's exchange
  // Tensor-core modes: the weights prepared once per optimizer step instead of once per product (same layout as
  // params): w_hi = TF32-rounded weights, w_lo = TF32-rounded remainder (3xTF32 only).
  float *w_hi = nullptr, *w_lo = nullptr; bool weights_prepared = false;
  // The split-K partial results of the three weight-gradient products and the row-slab partial sums of the three
  // bias gradients stay here until ONE kernel reduces all six into the flat gradient buffer.
  float* partials = nullptr; int64_t cap_w2 = 0, cap_w1 = 0, cap_wh = 0, cap_b = 0;
  float* loss_part = nullptr; int64_t cap_loss = 0;   // loss kernel's per-block partials: [blocks][2] {loss, kl} then [blocks][HP] column sums
  int64_t t = 0; int64_t steps_in_epoch = 0; int64_t last_launches = 0;
  std::vector<float> host_tmp;
  cudaStream_t copy_stream = nullptr;  // host->device staging of talos_ppo_update_host, overlapped with the steps
  std::vector<cudaEvent_t> chunk_ready; cudaEvent_t staging_free = nullptr;
};

namespace {

constexpr int MAX_STEPS_PER_EPOCH = 4096;

void gemm(talos_ctx* ctx, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
          int64_t ldb, float* C, int64_t ldc, int mode, const EpiArgs& e) {
  if (mode != TALOS_MODE_FP32 && talos_gemm_tc_launch(ctx, opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode, e)) return;
  talos_gemm_fp32_launch(ctx, opA, opB, M, N, K, A, lda, 0, B, ldb, 0, C, ldc, 0, 1, e);
}

// gemm() with the weight operand B taken from the prepared copies (when the mode uses them).
void gemm_w(talos_ppo* p, int opA, int opB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, int64_t w_off, int64_t ldb,
            float* C, int64_t ldc, const EpiArgs& e) {
  talos_ctx* ctx = p->ctx; const int mode = p->cfg.mode; const float* B = p->params + w_off;
  TcExtra x; if (p->w_hi) { x.b_hi = p->w_hi + w_off; x.b_lo = p->w_lo ? p->w_lo + w_off : nullptr; }
  if (mode != TALOS_MODE_FP32 && talos_gemm_tc_launch(ctx, opA, opB, M, N, K, A, lda, B, ldb, C, ldc, mode, e, &x)) return;
  talos_gemm_fp32_launch(ctx, opA, opB, M, N, K, A, lda, 0, B, ldb, 0, C, ldc, 0, 1, e);
}
// Weight-gradient product C = A^T.B that may leave its split-K partials in `partial` (returns their count, or 0 when
// C was written directly).
int gemm_dw(talos_ppo* p, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B, int64_t ldb, float* C, float* partial,
            int64_t cap) {
  talos_ctx* ctx = p->ctx; const int mode = p->cfg.mode; int splits = 1;
  EpiArgs none{nullptr, nullptr, 0, nullptr, 0, 0, 0, 0};
  TcExtra x; x.partial = partial; x.partial_floats = (size_t)cap; x.splits_out = &splits;
  if (mode != TALOS_MODE_FP32 && talos_gemm_tc_launch(ctx, 1, 0, M, N, K, A, lda, B, ldb, C, N, mode, none, &x)) return splits > 1 ? splits : 0;
  talos_gemm_fp32_launch(ctx, 1, 0, M, N, K, A, lda, 0, B, ldb, 0, C, N, 0, 1, none);
  return 0;
}

__global__ void prepare_weights_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float a = w[i];
  const float h = __uint_as_float((__float_as_uint(a) + 0x1000u) & 0xFFFFE000u);        // round to nearest TF32, ties away
  hi[i] = h;
  if (lo) lo[i] = __uint_as_float((__float_as_uint(a - h) + 0x1000u) & 0xFFFFE000u);
}
void ensure_weights_prepared(talos_ppo* p) {
  if (!p->w_hi || p->weights_prepared) return;
  prepare_weights_kernel<<<(unsigned)ceil_div(p->n_int, 256), 256, 0, p->ctx->stream>>>(p->params, p->w_hi, p->w_lo, p->n_int);
  talos_launched(p->ctx, "prepare_weights");
  p->weights_prepared = true;
}

// One launch for the whole flat gradient: segment s of `dst` (n elements) = sum over `slabs` partial rows of length n,
// added in a fixed order (eight slab lanes per column, each striding the slabs, then the eight lane sums in lane
// order): deterministic and independent of the launch geometry.  Segments with slabs = 0 were written directly.
// The seventh segment is the loss kernel's per-block {loss, kl} sums; its block also writes the sample count behind them.
constexpr int GRAD_SEGS = 7;
struct GradSegs { float* dst[GRAD_SEGS]; const float* src[GRAD_SEGS]; int n[GRAD_SEGS]; int slabs[GRAD_SEGS]; int first_block[GRAD_SEGS + 1]; float count; };
__global__ void __launch_bounds__(256)
grad_gather_kernel(GradSegs g) {
  __shared__ float sh[8][33];
  int s = 0;
  while (s < GRAD_SEGS - 1 && (int)blockIdx.x >= g.first_block[s + 1]) ++s;
  const int cl = threadIdx.x & 31, pl = threadIdx.x >> 5;
  const int c = ((int)blockIdx.x - g.first_block[s]) * 32 + cl;
  const int n = g.n[s], slabs = g.slabs[s];
  const float* src = g.src[s];
  float acc = 0.f;
  if (c < n) {
#pragma unroll 8
    for (int q = pl; q < slabs; q += 8) acc += src[(size_t)q * n + c];
  }
  sh[pl][cl] = acc;
  __syncthreads();
  if (pl == 0 && c < n) {
    float t = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) t += sh[l][cl];
    g.dst[s][c] = t;
  }
  if (s == GRAD_SEGS - 1 && threadIdx.x == 0) { g.dst[s][2] = g.count; g.dst[s][3] = 0.f; }       // {loss, kl, count, 0}: the tail of the flat gradient
}

__global__ void unpack_heads_kernel(const float* __restrict__ z, int HP, int A, long long n, float* __restrict__ logits, float* __restrict__ values) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * (A + 1)) return;
  long long r = i / (A + 1); int c = (int)(i % (A + 1));
  float v = z[r * HP + c];
  if (c < A) { if (logits) logits[r * A + c] = v; } else if (values) values[r] = v;
}
__global__ void log_prob_kernel(const float* __restrict__ z, int HP, int A, const int* __restrict__ actions, long long n, float* __restrict__ out,
                                int32_t* __restrict__ status) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* l = z + i * HP; float mx = -INFINITY;
  for (int a = 0; a < A; ++a) mx = fmaxf(mx, l[a]);
  float se = 0.f; for (int a = 0; a < A; ++a) se += expf(l[a] - mx);
  const int act = actions[i];
  if (act < 0 || act >= A) { atomicExch(status, TALOS_DEV_BAD_INDEX); out[i] = 0.f; return; }   // no read outside the row; reported at the next sync
  out[i] = l[act] - (logf(se) + mx);
}

void forward(talos_ppo* p, const float* obs, int64_t n) {
  const auto& c = p->cfg; const float* P = p->params;
  ensure_weights_prepared(p);
  EpiArgs e1{P + p->o_b1, nullptr, 0, nullptr, 0, TALOS_ACT_TANH, 0, 0};
  gemm_w(p, 0, 0, n, c.hidden, c.obs_dim, obs, c.obs_dim, p->o_w1, c.hidden, p->h1, c.hidden, e1);
  EpiArgs e2{P + p->o_b2, nullptr, 0, nullptr, 0, TALOS_ACT_TANH, 0, 0};
  gemm_w(p, 0, 0, n, c.hidden, c.hidden, p->h1, c.hidden, p->o_w2, c.hidden, p->h2, c.hidden, e2);
  EpiArgs e3{P + p->o_bh, nullptr, 0, nullptr, 0, 0, 0, 0};
  gemm_w(p, 0, 0, n, p->HP, c.hidden, p->h2, c.hidden, p->o_wh, p->HP, p->z, p->HP, e3);
}

void pack_params(talos_ppo* p, const float* canon, float* internal) {
  const auto& c = p->cfg; const int64_t H = c.hidden, O = c.obs_dim, A = c.n_actions;
  std::fill(internal, internal + p->n_int, 0.f);
  const float* s = canon;
  std::copy(s, s + O * H, internal + p->o_w1); s += O * H;
  std::copy(s, s + H, internal + p->o_b1); s += H;
  std::copy(s, s + H * H, internal + p->o_w2); s += H * H;
  std::copy(s, s + H, internal + p->o_b2); s += H;
  for (int64_t r = 0; r < H; ++r) for (int64_t a = 0; a < A; ++a) internal[p->o_wh + r * p->HP + a] = s[r * A + a];
  s += H * A;
  for (int64_t a = 0; a < A; ++a) internal[p->o_bh + a] = s[a];
  s += A;
  for (int64_t r = 0; r < H; ++r) internal[p->o_wh + r * p->HP + A] = s[r];
  s += H;
  internal[p->o_bh + A] = s[0];
}
void unpack_params(talos_ppo* p, const float* internal, float* canon) {
  const auto& c = p->cfg; const int64_t H = c.hidden, O = c.obs_dim, A = c.n_actions;
  float* d = canon;
  std::copy(internal + p->o_w1, internal + p->o_w1 + O * H, d); d += O * H;
  std::copy(internal + p->o_b1, internal + p->o_b1 + H, d); d += H;
  std::copy(internal + p->o_w2, internal + p->o_w2 + H * H, d); d += H * H;
  std::copy(internal + p->o_b2, internal + p->o_b2 + H, d); d += H;
  for (int64_t r = 0; r < H; ++r) for (int64_t a = 0; a < A; ++a) d[r * A + a] = internal[p->o_wh + r * p->HP + a];
  d += H * A;
  for (int64_t a = 0; a < A; ++a) d[a] = internal[p->o_bh + a];
  d += A;
  for (int64_t r = 0; r < H; ++r) d[r] = internal[p->o_wh + r * p->HP + A];
  d += H;
  d[0] = internal[p->o_bh + A];
}

void check(talos_ppo* p) { TALOS_REQUIRE(p != nullptr, TALOS_ERR_ARG, "null trainer"); talos_check_ctx(p->ctx); }

void step(talos_ppo* p, talos_comm* comm, const float* obs, const int32_t* actions, const float* old_logp, const float* adv,
          const float* ret, int64_t n) {
  const auto& c = p->cfg; talos_ctx* ctx = p->ctx; const float* P = p->params;
  // With the peer-memory exchange the step's gradient buffer IS this rank's exchange slot: the backward products write
  // straight into memory the other ranks have mapped, and one kernel does exchange + Adam + weight preparation.
  const bool peer = comm && comm->x.active && (size_t)(p->n_int + 4) <= comm->x.slot_floats && comm->ctx == ctx;
  const uint64_t seq = peer ? comm->x.seq + 1 : 0;
  float* G = peer ? comm->x.slot(comm->rank, seq) : p->grads;
  const int64_t H = c.hidden, HP = p->HP;
  const int64_t l0 = ctx->launches.load();
  float* tail = G + p->n_int;
  forward(p, obs, n);
  // per-sample loss and its gradient w.r.t. [logits | value]; sums (denominator 1), divided by the global count in Adam.
  // For the action counts the loss kernel is specialised for, it also leaves the heads' bias gradient (column sums of
  // its output) and the {loss, kl} sums as per-block partials for the gather kernel: no separate column-sum and
  // statistics launches, and the tail of the flat gradient is written rather than cleared and added to.
  talos_status st = TALOS_OK;
  const int loss_blocks = (int)ceil_div(n, 128);
  const bool loss_fused = p->loss_part && talos_ppo_loss_colsum_supported(c.n_actions, (int)HP) && (int64_t)loss_blocks * (2 + HP) <= p->cap_loss;
  float* loss_cs = p->loss_part ? p->loss_part + 2 * (size_t)loss_blocks : nullptr;
  if (loss_fused) {
    talos_ppo_loss_launch(ctx, p->z, HP, p->z + c.n_actions, HP, actions, old_logp, adv, ret, n, c.n_actions, c.clip, c.c_value, c.c_entropy, 1.0f,
                          p->dz, HP, p->dz + c.n_actions, HP, p->loss_part, loss_cs, (int)HP);
  } else {
    TALOS_CHECK_CUDA(cudaMemsetAsync(tail, 0, 4 * sizeof(float), ctx->stream));    // Adam::zero_grad (src/ppo.rs:686); GEMMs overwrite the rest
    st = talos_ppo_loss_fwd_bwd(ctx, p->z, HP, p->z + c.n_actions, HP, actions, old_logp, adv, ret, n, c.n_actions, c.clip,
                                c.c_value, c.c_entropy, 1.0f, p->dz, HP, p->dz + c.n_actions, HP, tail);
    if (st) throw talos_error(st, talos_last_error_string());
  }
  EpiArgs none{nullptr, nullptr, 0, nullptr, 0, 0, 0, 0};
  // Each gradient is either written straight into G or left as partial sums (split-K slabs of a weight-gradient
  // product, row-slab column sums of a bias gradient) that ONE gather kernel reduces into G at the end, instead of
  // six small reduction launches.
  float* part_w2 = p->partials; float* part_w1 = part_w2 + p->cap_w2; float* part_wh = part_w1 + p->cap_w1;
  float* part_b2 = part_wh + p->cap_wh; float* part_b1 = part_b2 + p->cap_b; float* part_bh = part_b1 + p->cap_b;
  GradSegs gs{};
  auto seg = [&](int i, float* dst, const float* src, int64_t count, int slabs) { gs.dst[i] = dst; gs.src[i] = src; gs.n[i] = (int)count; gs.slabs[i] = slabs; };
  // column sums of `dy` (times tanh'(h_saved) in place when h_saved is given): partial slabs, or directly into db
  auto bias_grad = [&](int i, float* dy, const float* h_saved, int64_t width, float* db, float* part) {
    int slabs = p->partials ? talos_colsum_partials_launch(ctx, dy, dy, h_saved, h_saved ? TALOS_ACT_TANH : 0, n, width, part, p->cap_b) : 0;
    if (slabs == 0) {
      if (h_saved) { if (!talos_dact_colsum_launch(ctx, dy, dy, h_saved, TALOS_ACT_TANH, db, n, width, 0)) throw talos_error(TALOS_ERR_CUDA, "dact + colsum kernel refused an aligned shape"); }
      else { talos_status s2 = talos_colsum(ctx, dy, db, n, width, 0); if (s2) throw talos_error(s2, talos_last_error_string()); }
    }
    seg(i, db, part, width, slabs);
  };
  // dH = (dZ_next . W^T) * tanh'(h), db = colsum(dH).  The tanh' factor is not fused into the GEMM's epilogue when
  // the streaming kernel can take it: that epilogue reads the saved activation row by row and is what bounds these
  // skinny GEMMs (72 -> ~30 us at K = 32); one streaming pass applies the factor in place and produces the bias
  // gradient's column sums at the same time.
  auto backprop_hidden = [&](int i, const float* dz_next, int64_t k, int64_t w_off, float* dh, const float* h_saved, float* db, float* part) {
    if (H % 4 == 0 && H <= 1024) {                                              // what the streaming kernel takes (buffers are aligned)
      // The tensor-core modes take the factor and the column sums into the GEMM's own epilogue, which fetches the saved
      // activation tiles by TMA: no streaming pass at all (the launcher says whether the shape qualified).
      if (p->partials && p->w_hi && (p->cfg.mode == TALOS_MODE_TF32X3 || p->cfg.mode == TALOS_MODE_TF32)) {
        int slabs = 0;
        TcExtra x; x.b_hi = p->w_hi + w_off; x.b_lo = p->w_lo ? p->w_lo + w_off : nullptr;
        x.tanh_saved = h_saved; x.ld_saved = H; x.colsum_part = part; x.colsum_floats = (size_t)p->cap_b; x.colsum_slabs_out = &slabs;
        if (talos_gemm_tc_launch(ctx, 0, 1, n, H, k, dz_next, k, p->params + w_off, k, dh, H, p->cfg.mode, none, &x)) {
          if (slabs > 0) seg(i, db, part, H, slabs); else bias_grad(i, dh, h_saved, H, db, part);
          return;
        }
      }
      gemm_w(p, 0, 1, n, H, k, dz_next, k, w_off, k, dh, H, none);
      bias_grad(i, dh, h_saved, H, db, part);
      return;
    }
    EpiArgs d{nullptr, nullptr, 0, h_saved, H, 0, TALOS_ACT_TANH, 0};
    gemm_w(p, 0, 1, n, H, k, dz_next, k, w_off, k, dh, H, d);
    bias_grad(i, dh, nullptr, H, db, part);
  };
  // heads: dWh = h2^T.dz ; dbh = colsum(dz) ; dh2 = (dz.Wh^T) * (1 - h2^2)
  seg(0, G + p->o_wh, part_wh, H * HP, gemm_dw(p, H, HP, n, p->h2, H, p->dz, HP, G + p->o_wh, p->partials ? part_wh : nullptr, p->cap_wh));
  if (loss_fused) { seg(1, G + p->o_bh, loss_cs, HP, loss_blocks); seg(6, tail, p->loss_part, 2, loss_blocks); gs.count = (float)n; }
  else bias_grad(1, p->dz, nullptr, HP, G + p->o_bh, part_bh);
  backprop_hidden(2, p->dz, HP, p->o_wh, p->dh2, p->h2, G + p->o_b2, part_b2);
  // layer 2
  seg(3, G + p->o_w2, part_w2, H * H, gemm_dw(p, H, H, n, p->h1, H, p->dh2, H, G + p->o_w2, p->partials ? part_w2 : nullptr, p->cap_w2));
  backprop_hidden(4, p->dh2, H, p->o_w2, p->dh1, p->h1, G + p->o_b1, part_b1);
  // layer 1 (no gradient w.r.t. the observations)
  seg(5, G + p->o_w1, part_w1, c.obs_dim * H, gemm_dw(p, c.obs_dim, H, n, obs, c.obs_dim, p->dh1, H, G + p->o_w1, p->partials ? part_w1 : nullptr, p->cap_w1));
  {
    int blocks = 0;
    for (int i = 0; i < GRAD_SEGS; ++i) { gs.first_block[i] = blocks; if (gs.slabs[i] > 0) blocks += (int)ceil_div(gs.n[i], 32); }
    gs.first_block[GRAD_SEGS] = blocks;
    if (blocks > 0) { grad_gather_kernel<<<blocks, 256, 0, ctx->stream>>>(gs); talos_launched(ctx, "grad_gather"); }
  }
  p->t += 1;
  float* stat_slot = p->step_stats + 4 * (p->steps_in_epoch % MAX_STEPS_PER_EPOCH);
  // One kernel applies the step: sum of the ranks' gradient slots in rank order (over peer memory when there are peers;
  // a single rank "sums" its own buffer), Adam, and the TF32-prepared copies of the new weights.  Only the NCCL route
  // (peers that could not map each other's memory) needs the separate all-reduce + Adam + preparation launches.
  const bool fused_update = peer || (!comm && p->n_int % 4 == 0);
  if (fused_update) {
    XchgAdamArgs a{};
    if (peer) {
      for (int r = 0; r < comm->nranks; ++r) { a.slot[r] = comm->x.slot(r, seq); a.peer_flags[r] = comm->x.flags(r); }
      a.world = comm->nranks; a.rank = comm->rank; a.seq = seq; a.spins = comm->x.wait_spins; a.skip_signal = comm->x.dbg_skip_signal;
    } else {
      a.slot[0] = G; a.peer_flags[0] = nullptr; a.world = 1; a.rank = 0; a.seq = 0; a.skip_signal = 1;     // nobody to signal, nobody to wait for
    }
    a.status = ctx->dev_status; a.params = p->params; a.m = p->m; a.v = p->v; a.w_hi = p->w_hi; a.w_lo = p->w_lo; a.grads_out = p->grads; a.stats_out = stat_slot;
    a.n = p->n_int; a.lr = c.lr; a.b1 = c.beta1; a.b2 = c.beta2; a.eps = c.eps;
    a.inv_bc1 = (float)(1.0 / (1.0 - pow((double)c.beta1, (double)p->t))); a.inv_bc2 = (float)(1.0 / (1.0 - pow((double)c.beta2, (double)p->t)));
    talos_xchg_adam_launch(ctx, a);
    if (peer) { comm->x.seq = seq; comm->x.dbg_skip_signal = 0; }
    p->weights_prepared = p->w_hi != nullptr;
  } else {
    if (comm) { if ((st = talos_comm_allreduce_sum(comm, G, p->n_int + 4))) throw talos_error(st, talos_last_error_string()); }
    talos_adam_launch(ctx, p->params, G, p->m, p->v, p->n_int, p->t, c.lr, c.beta1, c.beta2, c.eps, 1.0f, tail + 2, 0.f, stat_slot);
    p->weights_prepared = false;
    ensure_weights_prepared(p);                                // for the next step's products (and the caller's next forward)
  }
  p->steps_in_epoch += 1;
  p->last_launches = ctx->launches.load() - l0;
}

// `ready` (optional): one event per minibatch that the first epoch's step must wait for (its transitions are
// still being copied in on another stream).
void update(talos_ppo* p, talos_comm* comm, const float* obs, const int32_t* actions, const float* old_logp, const float* adv,
            const float* ret, int64_t N, int32_t epochs, float kl_stop, float* epoch_kl, int32_t* epochs_run,
            const std::vector<cudaEvent_t>* ready = nullptr, const std::function<void(int64_t)>* stage_chunk = nullptr) {
  const int64_t mb = p->cfg.minibatch;
  int32_t done = 0;
  std::vector<float> stats;
  const int64_t steps_per_epoch = (N + mb - 1) / mb;
  TALOS_REQUIRE(steps_per_epoch <= MAX_STEPS_PER_EPOCH, TALOS_ERR_UNSUPPORTED, "too many minibatches per epoch");
  // With the early stop disabled nothing on the host depends on an epoch's KL before the next epoch starts, so the
  // per-step statistics of ALL epochs are read back once at the end and the stream never drains in between (each drain
  // costs the launch queue's refill, tens of microseconds).  With the stop enabled (the reference's behaviour,
  // src/ppo.rs:762-767) every epoch ends with the read-back it needs.
  const bool defer = !(kl_stop > 0.f) && (int64_t)epochs * steps_per_epoch <= MAX_STEPS_PER_EPOCH;
  auto epoch_mean_kl = [&](const float* st, int64_t steps) {
    double kl = 0, cnt = 0;
    for (int64_t i = 0; i < steps; ++i) { kl += st[4 * i + 1]; cnt += st[4 * i + 2]; }
    return cnt > 0 ? (float)(kl / cnt) : 0.f;
  };
  p->steps_in_epoch = 0;
  for (int32_t e = 0; e < epochs; ++e) {
    if (!defer) p->steps_in_epoch = 0;                       // (deferred: the slots of later epochs follow the earlier ones)
    for (int64_t s = 0; s < N; s += mb) {
      int64_t n = std::min(mb, N - s);
      if (ready && e == 0) TALOS_CHECK_CUDA(cudaStreamWaitEvent(p->ctx->stream, (*ready)[(size_t)(s / mb)], 0));
      step(p, comm, obs + s * p->cfg.obs_dim, actions + s, old_logp + s, adv + s, ret + s, n);
      if (stage_chunk && e == 0) (*stage_chunk)(s / mb + 2);           // keep the copy stream two minibatches ahead of the steps
    }
    done = e + 1;
    if (defer) continue;
    // mean approx-KL of the epoch (src/ppo.rs:729-731, :762-767): the step's device->host read
    stats.resize(4 * (size_t)p->steps_in_epoch);
    TALOS_CHECK_CUDA(cudaMemcpyAsync(stats.data(), p->step_stats, stats.size() * sizeof(float), cudaMemcpyDeviceToHost, p->ctx->stream));
    talos_sync_and_check(p->ctx);        // a kernel that gave up (or met a bad action) ends the update here: no further epochs on garbage gradients
    const float mean_kl = epoch_mean_kl(stats.data(), p->steps_in_epoch);
    if (epoch_kl) epoch_kl[e] = mean_kl;
    if (kl_stop > 0.f && mean_kl > kl_stop * 1.5f) break;
  }
  if (defer) {
    stats.resize(4 * (size_t)p->steps_in_epoch);
    TALOS_CHECK_CUDA(cudaMemcpyAsync(stats.data(), p->step_stats, stats.size() * sizeof(float), cudaMemcpyDeviceToHost, p->ctx->stream));
    talos_sync_and_check(p->ctx);
    for (int32_t e = 0; e < done; ++e) if (epoch_kl) epoch_kl[e] = epoch_mean_kl(stats.data() + 4 * (size_t)(e * steps_per_epoch), steps_per_epoch);
  }
  if (epochs_run) *epochs_run = done;
}

}  // namespace

TALOS_API talos_status talos_ppo_create(talos_ctx* ctx, const talos_ppo_config* cfg, talos_ppo** out) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(cfg && out, TALOS_ERR_ARG, "null pointer");
  TALOS_REQUIRE(cfg->obs_dim >= 1 && cfg->hidden >= 1 && cfg->n_actions >= 1 && cfg->n_actions <= 63 && cfg->minibatch >= 1,
                TALOS_ERR_SHAPE, "bad PPO configuration");
  TALOS_REQUIRE(cfg->mode >= TALOS_MODE_FP32 && cfg->mode <= TALOS_MODE_TF32, TALOS_ERR_ARG, "bad mode");
  talos_ppo* p = new talos_ppo();
  p->ctx = ctx; p->cfg = *cfg;
  const int64_t H = cfg->hidden, O = cfg->obs_dim, mb = cfg->minibatch;
  p->HP = cfg->n_actions + 1 <= 32 ? 32 : 64;
  auto up4 = [](int64_t x) { return (x + 3) & ~int64_t(3); };     // keep every matrix 16-byte aligned for TMA
  int64_t o = 0;
  p->o_w1 = o; o = up4(o + O * H); p->o_b1 = o; o = up4(o + H); p->o_w2 = o; o = up4(o + H * H); p->o_b2 = o; o = up4(o + H);
  p->o_wh = o; o = up4(o + H * p->HP); p->o_bh = o; o = up4(o + p->HP);
  p->n_int = o;
  auto alloc = [&](float** ptr, int64_t n) {
    cudaError_t e = cudaMalloc(ptr, sizeof(float) * (size_t)n);
    if (e != cudaSuccess) { cudaGetLastError(); throw talos_error(TALOS_ERR_ALLOC, "PPO buffer allocation failed"); }
    TALOS_CHECK_CUDA(cudaMemsetAsync(*ptr, 0, sizeof(float) * (size_t)n, ctx->stream));
  };
  alloc(&p->params, p->n_int); alloc(&p->grads, p->n_int + 4); alloc(&p->m, p->n_int); alloc(&p->v, p->n_int);
  alloc(&p->h1, mb * H); alloc(&p->h2, mb * H); alloc(&p->dh1, mb * H); alloc(&p->dh2, mb * H);
  alloc(&p->z, mb * p->HP); alloc(&p->dz, mb * p->HP);
  alloc(&p->step_stats, 4 * MAX_STEPS_PER_EPOCH);
  p->cap_loss = up4(ceil_div(mb, 128) * (2 + p->HP)); alloc(&p->loss_part, p->cap_loss);
  if (cfg->mode != TALOS_MODE_FP32) {
    alloc(&p->w_hi, p->n_int);
    if (cfg->mode == TALOS_MODE_TF32X3) alloc(&p->w_lo, p->n_int);
    // room for the largest split count the GEMM launcher picks: one slab per 512 reduction elements in 3xTF32 mode
    // (never more than that), at most one per SM otherwise
    const int64_t max_splits = std::max<int64_t>(ctx->sm_count, mb / 512 + 1) + 1;
    p->cap_w2 = up4(max_splits * H * H); p->cap_w1 = up4(max_splits * O * H); p->cap_wh = up4(max_splits * H * p->HP);
    p->cap_b = up4((4 * (int64_t)ctx->sm_count + 1) * std::max<int64_t>(H, p->HP));
    alloc(&p->partials, p->cap_w2 + p->cap_w1 + p->cap_wh + 3 * p->cap_b);
  }
  *out = p;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_destroy(talos_ppo* p) {
  TALOS_ENTRY_BEGIN
  if (!p) return TALOS_OK;
  cudaSetDevice(p->ctx->device); cudaStreamSynchronize(p->ctx->stream);
  for (float* q : {p->params, p->grads, p->m, p->v, p->h1, p->h2, p->dh1, p->dh2, p->z, p->dz, p->step_stats, p->w_hi, p->w_lo, p->partials, p->loss_part}) cudaFree(q);
  for (cudaEvent_t ev : p->chunk_ready) cudaEventDestroy(ev);
  if (p->staging_free) cudaEventDestroy(p->staging_free);
  if (p->copy_stream) cudaStreamDestroy(p->copy_stream);
  delete p;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_param_count(talos_ppo* p, int64_t* n_out) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(p && n_out, TALOS_ERR_ARG, "null pointer");
  const auto& c = p->cfg;
  *n_out = (int64_t)c.obs_dim * c.hidden + c.hidden + (int64_t)c.hidden * c.hidden + c.hidden + (int64_t)c.hidden * c.n_actions +
           c.n_actions + c.hidden + 1;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_set_params_host(talos_ppo* p, const float* flat) {
  TALOS_ENTRY_BEGIN
  check(p); TALOS_REQUIRE(flat != nullptr, TALOS_ERR_ARG, "null pointer");
  p->host_tmp.resize((size_t)p->n_int);
  pack_params(p, flat, p->host_tmp.data());
  TALOS_CHECK_CUDA(cudaMemcpyAsync(p->params, p->host_tmp.data(), sizeof(float) * (size_t)p->n_int, cudaMemcpyHostToDevice, p->ctx->stream));
  TALOS_CHECK_CUDA(cudaStreamSynchronize(p->ctx->stream));
  p->weights_prepared = false;
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ppo_get_params_host(talos_ppo* p, float* flat) {
  TALOS_ENTRY_BEGIN
  check(p); TALOS_REQUIRE(flat != nullptr, TALOS_ERR_ARG, "null pointer");
  p->host_tmp.resize((size_t)p->n_int);
  TALOS_CHECK_CUDA(cudaMemcpyAsync(p->host_tmp.data(), p->params, sizeof(float) * (size_t)p->n_int, cudaMemcpyDeviceToHost, p->ctx->stream));
  talos_sync_and_check(p->ctx);
  unpack_params(p, p->host_tmp.data(), flat);
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ppo_get_grads_host(talos_ppo* p, float* flat) {
  TALOS_ENTRY_BEGIN
  check(p); TALOS_REQUIRE(flat != nullptr, TALOS_ERR_ARG, "null pointer");
  TALOS_REQUIRE(p->t > 0, TALOS_ERR_ARG, "no optimizer step has run");
  p->host_tmp.resize((size_t)p->n_int + 4);
  TALOS_CHECK_CUDA(cudaMemcpyAsync(p->host_tmp.data(), p->grads, sizeof(float) * (size_t)(p->n_int + 4), cudaMemcpyDeviceToHost, p->ctx->stream));
  talos_sync_and_check(p->ctx);
  const float count = std::max(p->host_tmp[(size_t)p->n_int + 2], 1.f);       // the buffer holds sums over the samples of all ranks
  for (int64_t i = 0; i < p->n_int; ++i) p->host_tmp[(size_t)i] /= count;
  unpack_params(p, p->host_tmp.data(), flat);
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ppo_reset_optimizer(talos_ppo* p) {
  TALOS_ENTRY_BEGIN
  check(p);
  TALOS_CHECK_CUDA(cudaMemsetAsync(p->m, 0, sizeof(float) * (size_t)p->n_int, p->ctx->stream));
  TALOS_CHECK_CUDA(cudaMemsetAsync(p->v, 0, sizeof(float) * (size_t)p->n_int, p->ctx->stream));
  p->t = 0;
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ppo_set_lr(talos_ppo* p, float lr) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(p != nullptr, TALOS_ERR_ARG, "null trainer"); p->cfg.lr = lr;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_forward(talos_ppo* p, const float* obs, int64_t n, float* logits_out, float* values_out) {
  TALOS_ENTRY_BEGIN
  check(p); TALOS_REQUIRE(n >= 0 && (obs || n == 0), TALOS_ERR_ARG, "bad observations");
  const auto& c = p->cfg;
  for (int64_t s = 0; s < n; s += c.minibatch) {
    int64_t m = std::min<int64_t>(c.minibatch, n - s);
    forward(p, obs + s * c.obs_dim, m);
    int64_t total = m * (c.n_actions + 1);
    unpack_heads_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, p->ctx->stream>>>(p->z, p->HP, c.n_actions, m, logits_out ? logits_out + s * c.n_actions : nullptr,
                                                                                     values_out ? values_out + s : nullptr);
    talos_launched(p->ctx, "unpack_heads");
  }
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ppo_log_prob(talos_ppo* p, const float* obs, const int32_t* actions, int64_t n, float* out) {
  TALOS_ENTRY_BEGIN
  check(p); TALOS_REQUIRE(n >= 0 && ((obs && actions && out) || n == 0), TALOS_ERR_ARG, "null pointer");
  const auto& c = p->cfg;
  for (int64_t s = 0; s < n; s += c.minibatch) {
    int64_t m = std::min<int64_t>(c.minibatch, n - s);
    forward(p, obs + s * c.obs_dim, m);
    log_prob_kernel<<<(unsigned)ceil_div(m, 256), 256, 0, p->ctx->stream>>>(p->z, p->HP, c.n_actions, actions + s, m, out + s, p->ctx->dev_status);
    talos_launched(p->ctx, "log_prob");
  }
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_step(talos_ppo* p, talos_comm* comm, const float* obs, const int32_t* actions,
                                      const float* old_logp, const float* adv, const float* ret, int64_t n) {
  TALOS_ENTRY_BEGIN
  check(p);
  TALOS_REQUIRE(n >= 1 && n <= p->cfg.minibatch, TALOS_ERR_SHAPE, "minibatch larger than configured");
  TALOS_REQUIRE(obs && actions && old_logp && adv && ret, TALOS_ERR_ARG, "null pointer");
  step(p, comm, obs, actions, old_logp, adv, ret, n);
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_update(talos_ppo* p, talos_comm* comm, const float* obs, const int32_t* actions,
                                        const float* old_logp, const float* adv, const float* ret, int64_t N, int32_t epochs,
                                        float kl_stop, float* epoch_kl_host, int32_t* epochs_run_out) {
  TALOS_ENTRY_BEGIN
  check(p);
  TALOS_REQUIRE(N >= 0 && epochs >= 0, TALOS_ERR_SHAPE, "bad update size");
  if (N == 0) { if (epochs_run_out) *epochs_run_out = 0; return TALOS_OK; }     // empty memory: nothing to do (src/ppo.rs:626-628)
  TALOS_REQUIRE(obs && actions && old_logp && adv && ret, TALOS_ERR_ARG, "null pointer");
  update(p, comm, obs, actions, old_logp, adv, ret, N, epochs, kl_stop, epoch_kl_host, epochs_run_out);
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_update_host(talos_ppo* p, talos_comm* comm, const float* obs_h, const int32_t* actions_h,
                                             const float* old_logp_h, const float* adv_h, const float* ret_h, int64_t N,
                                             int32_t epochs, float kl_stop, float* epoch_kl_host, int32_t* epochs_run_out) {
  TALOS_ENTRY_BEGIN
  check(p);
  TALOS_REQUIRE(N >= 0 && epochs >= 0, TALOS_ERR_SHAPE, "bad update size");
  if (N == 0) { if (epochs_run_out) *epochs_run_out = 0; return TALOS_OK; }
  TALOS_REQUIRE(obs_h && actions_h && old_logp_h && adv_h && ret_h, TALOS_ERR_ARG, "null pointer");
  const int64_t O = p->cfg.obs_dim;
  size_t bytes = sizeof(float) * (size_t)(N * O) + 4 * sizeof(float) * (size_t)N + 1024;
  char* base = (char*)talos_workspace2(p->ctx, bytes);
  float* obs = (float*)base; int32_t* actions = (int32_t*)(obs + N * O);
  float* old_logp = (float*)(actions + N); float* adv = old_logp + N; float* ret = adv + N;
  // Copies run minibatch by minibatch on their own stream; the step on minibatch i waits only for chunk i, so
  // the transfer of chunk i+1 overlaps the compute of chunk i (pinned host memory makes the copies asynchronous).
  if (!p->copy_stream) {
    TALOS_CHECK_CUDA(cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking));
    TALOS_CHECK_CUDA(cudaEventCreateWithFlags(&p->staging_free, cudaEventDisableTiming));
  }
  const int64_t mb = p->cfg.minibatch, chunks = (N + mb - 1) / mb;
  while ((int64_t)p->chunk_ready.size() < chunks) {
    cudaEvent_t ev; TALOS_CHECK_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)); p->chunk_ready.push_back(ev);
  }
  cudaStream_t cs = p->copy_stream;
  TALOS_CHECK_CUDA(cudaEventRecord(p->staging_free, p->ctx->stream));        // earlier work may still read the staging buffer
  TALOS_CHECK_CUDA(cudaStreamWaitEvent(cs, p->staging_free, 0));
  // The copies of minibatch c are enqueued when step c - 2 has been launched (the first two up front), not all at the
  // start: enqueueing 5 copies per minibatch for the whole shard first would hold back the first step's launch by the
  // host time of all of them.
  const std::function<void(int64_t)> stage_chunk = [&](int64_t c) {
    if (c >= chunks) return;
    const int64_t s0 = c * mb, n = std::min(mb, N - s0);
    TALOS_CHECK_CUDA(cudaMemcpyAsync(obs + s0 * O, obs_h + s0 * O, sizeof(float) * (size_t)(n * O), cudaMemcpyHostToDevice, cs));
    TALOS_CHECK_CUDA(cudaMemcpyAsync(actions + s0, actions_h + s0, sizeof(int32_t) * (size_t)n, cudaMemcpyHostToDevice, cs));
    TALOS_CHECK_CUDA(cudaMemcpyAsync(old_logp + s0, old_logp_h + s0, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, cs));
    TALOS_CHECK_CUDA(cudaMemcpyAsync(adv + s0, adv_h + s0, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, cs));
    TALOS_CHECK_CUDA(cudaMemcpyAsync(ret + s0, ret_h + s0, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, cs));
    TALOS_CHECK_CUDA(cudaEventRecord(p->chunk_ready[(size_t)c], cs));
  };
  stage_chunk(0); stage_chunk(1);
  if (epochs == 0) for (int64_t c = 2; c < chunks; ++c) stage_chunk(c);       // (no steps to ride on: nothing to do, but leave the buffers consistent)
  update(p, comm, obs, actions, old_logp, adv, ret, N, epochs, kl_stop, epoch_kl_host, epochs_run_out, &p->chunk_ready, &stage_chunk);
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ppo_last_loss(talos_ppo* p, float* loss_out) {
  TALOS_ENTRY_BEGIN
  check(p); TALOS_REQUIRE(loss_out != nullptr, TALOS_ERR_ARG, "null pointer");
  TALOS_REQUIRE(p->steps_in_epoch > 0, TALOS_ERR_ARG, "no optimizer step has run");
  float s[4];
  TALOS_CHECK_CUDA(cudaMemcpyAsync(s, p->step_stats + 4 * ((p->steps_in_epoch - 1) % MAX_STEPS_PER_EPOCH), sizeof(s), cudaMemcpyDeviceToHost, p->ctx->stream));
  talos_sync_and_check(p->ctx);
  *loss_out = s[2] > 0 ? s[0] / s[2] : 0.f;
  TALOS_ENTRY_END
}
TALOS_API int64_t talos_ppo_launches_per_step(talos_ppo* p) { return p ? p->last_launches : 0; }
