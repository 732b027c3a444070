/*
 * talos_b200 -- C ABI of the data-parallel PPO actor-critic update (the training hot loop of
 * PPO::update, src/ppo.rs:625-770) and of the gradient exchange it needs on more than one GPU.
 *
 * The policy is the actor-critic split of src/ppo.rs:247-307 on an MLP trunk:
 *   h1 = tanh(obs.W1 + b1), h2 = tanh(h1.W2 + b2), logits = h2.Wp + bp, value = h2.Wv + bv.
 * One optimizer step = one minibatch: zero_grad -> per-sample loss (src/ppo.rs:702-752) ->
 * backward -> [allreduce over ranks] -> Adam::step (src/ppo.rs:519-533).  Minibatches are
 * consecutive, unshuffled index chunks (src/ppo.rs:681-685).
 */
#ifndef TALOS_B200_PPO_H
#define TALOS_B200_PPO_H

#include "talos_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct talos_ppo talos_ppo;
typedef struct talos_comm talos_comm;

typedef struct talos_ppo_config {
  int32_t obs_dim;      /* 64 in the benchmark config; DIM = 8 in the reference (src/neural.rs:3) */
  int32_t hidden;       /* 256 */
  int32_t n_actions;    /* 16; ACTION_SPACE = 5 in the reference (src/ppo.rs:15) */
  int32_t minibatch;    /* samples per optimizer step on this GPU */
  int32_t mode;         /* TALOS_MODE_* of the matrix products */
  float clip;           /* CLIP_EPSILON 0.2  (src/ppo.rs:17) */
  float c_value;        /* VALUE_COEF 0.5    (src/ppo.rs:20) */
  float c_entropy;      /* ENTROPY_COEF 0.01 (src/ppo.rs:21) */
  float lr;             /* 3e-4 (src/ppo.rs:567) */
  float beta1, beta2, eps;   /* 0.9, 0.999, 1e-8 (src/ppo.rs:509-511) */
} talos_ppo_config;

/* ---- gradient exchange: one NCCL all-reduce per optimizer step ------------------------------ */
/* Rank 0 calls talos_comm_unique_id and hands the 128 bytes to the other ranks by any host channel. */
talos_status talos_comm_unique_id(uint8_t* id_out_host);
talos_status talos_comm_init(talos_ctx* ctx, const uint8_t* id_host, int32_t nranks, int32_t rank, talos_comm** out);
talos_status talos_comm_destroy(talos_comm* comm);
/* In-place sum over ranks of n floats, enqueued on the ctx stream. */
talos_status talos_comm_allreduce_sum(talos_comm* comm, float* buf, int64_t n);
/* 1 when the ranks of this communicator (one node, NVLink) have mapped each other's exchange areas, so that
 * talos_ppo_step exchanges gradients with ONE kernel over peer memory -- publish, bounded wait, sum in rank order, Adam,
 * weight preparation -- instead of an NCCL all-reduce followed by two more kernels; 0 when that could not be set up on
 * some rank (or TALOS_COMM_NO_P2P is set) and the NCCL all-reduce serves.  The reference has no counterpart: it is a
 * single process. */
int32_t talos_comm_peer_exchange_active(talos_comm* comm);
/* Test hook: skip_next_signal != 0 makes THIS rank leave out its publication in the next peer-memory exchange, so that
 * the other ranks' bounded waits (wait_spins polls, 0 = default, else >= 1024) run out: they return by themselves,
 * raise their context's error word (TALOS_ERR_TIMEOUT at the next blocking call) and leave their parameters untouched.
 * Nothing faults or hangs.  The communicator must be destroyed afterwards (the ranks no longer agree). */
talos_status talos_debug_comm_stall(talos_comm* comm, int32_t skip_next_signal, uint32_t wait_spins);

/* ---- trainer --------------------------------------------------------------------------------- */
talos_status talos_ppo_create(talos_ctx* ctx, const talos_ppo_config* cfg, talos_ppo** out);
talos_status talos_ppo_destroy(talos_ppo* p);
/* Number of parameters in the canonical flat order
 *   W1[obs,hidden] b1[hidden] W2[hidden,hidden] b2[hidden] Wp[hidden,A] bp[A] Wv[hidden,1] bv[1]
 * (ActorCritic::parameters order, src/ppo.rs:302-307). */
talos_status talos_ppo_param_count(talos_ppo* p, int64_t* n_out);
talos_status talos_ppo_set_params_host(talos_ppo* p, const float* flat_host);
talos_status talos_ppo_get_params_host(talos_ppo* p, float* flat_host);
/* The gradient the last optimizer step applied: d(mean loss)/d(parameter) over the samples of all ranks, in the same
 * canonical order (what Tensor.grad holds after loss.backward(), src/ppo.rs:756-758).  Blocks. */
talos_status talos_ppo_get_grads_host(talos_ppo* p, float* flat_host);
/* Resets the Adam moments and the step counter (Adam::new, src/ppo.rs:494-513). */
talos_status talos_ppo_reset_optimizer(talos_ppo* p);
talos_status talos_ppo_set_lr(talos_ppo* p, float lr);

/* Policy evaluation on device data: logits [n,A] and values [n] (either may be NULL). */
talos_status talos_ppo_forward(talos_ppo* p, const float* obs, int64_t n, float* logits_out, float* values_out);
/* log pi(a|s) of the given actions under the current weights: what a rollout stores as the
 * old log-probability (src/ppo.rs:346). */
talos_status talos_ppo_log_prob(talos_ppo* p, const float* obs, const int32_t* actions, int64_t n, float* out);

/* One optimizer step on one minibatch of device-resident transitions (n <= cfg.minibatch).
 * comm may be NULL (single GPU).  Gradients are summed over the samples of all ranks and divided
 * by the global sample count, so G ranks x n samples equal one rank x G*n samples. */
talos_status talos_ppo_step(talos_ppo* p, talos_comm* comm, const float* obs, const int32_t* actions,
                            const float* old_logp, const float* adv, const float* ret, int64_t n);

/* The optimisation loops of PPO::update (src/ppo.rs:680-769) over N device-resident transitions:
 * `epochs` passes of consecutive minibatches.  kl_stop > 0 enables the early stop at mean
 * approx-KL > 1.5*kl_stop (0.015 in the reference, :678, :764).  epoch_kl_host (nullable) receives
 * the mean KL of each epoch run; epochs_run_out (nullable) the number of epochs executed. */
talos_status talos_ppo_update(talos_ppo* p, talos_comm* comm, const float* obs, const int32_t* actions,
                              const float* old_logp, const float* adv, const float* ret, int64_t N, int32_t epochs,
                              float kl_stop, float* epoch_kl_host, int32_t* epochs_run_out);
/* Same, from HOST buffers: the transitions are copied to the device inside the call (the end-to-end
 * path a host caller with rollout data in RAM uses). */
talos_status talos_ppo_update_host(talos_ppo* p, talos_comm* comm, const float* obs_host, const int32_t* actions_host,
                                   const float* old_logp_host, const float* adv_host, const float* ret_host, int64_t N,
                                   int32_t epochs, float kl_stop, float* epoch_kl_host, int32_t* epochs_run_out);
/* Mean loss of the last optimizer step (blocks until the step has finished). */
talos_status talos_ppo_last_loss(talos_ppo* p, float* loss_out);
/* Kernels launched by the last talos_ppo_step. */
int64_t talos_ppo_launches_per_step(talos_ppo* p);

#ifdef __cplusplus
}
#endif
#endif /* TALOS_B200_PPO_H */
