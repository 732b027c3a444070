// Internal view of a communicator: the NCCL handle plus, when the ranks could map each other's memory, the peer-memory
// exchange area used by the fused gradient-exchange + Adam kernel of the PPO trainer.
#pragma once
#include "common.cuh"
#include "../../include/talos_b200_ppo.h"

constexpr int TALOS_MAX_RANKS = 16;

// Layout of every rank's exchange area (one cudaMalloc, mapped into every peer through CUDA IPC):
//   [0, 1024)            flags: flags[r] = sequence number of the last exchange rank r has published (written BY rank r
//                        into EVERY rank's area, its own included), 8 bytes each
//   [1024, 1024 + 2*S)   two gradient slots of S bytes, used alternately (slot = sequence number & 1)
struct talos_xchg {
  bool active = false;
  size_t slot_floats = 0;                         // capacity of one slot
  char* local = nullptr;                          // this rank's area
  char* peer[TALOS_MAX_RANKS] = {nullptr};        // every rank's area as mapped here (peer[rank] == local)
  uint64_t seq = 0;                               // exchanges done so far (identical on every rank)
  unsigned wait_spins = 0;                        // 0: default poll limit; a test may shorten it
  int dbg_skip_signal = 0;                        // test hook: this rank leaves out its next publication
  float* slot(int r, uint64_t s) const { return (float*)(peer[r] + 1024 + (s & 1) * slot_floats * sizeof(float)); }
  unsigned long long* flags(int r) const { return (unsigned long long*)peer[r]; }
};

struct talos_comm {
  talos_ctx* ctx; void* nccl; int nranks, rank;
  talos_xchg x;
};

// Arguments of the fused kernel: sum the ranks' gradient slots in rank order, Adam, prepared weights.
struct XchgAdamArgs {
  const float* slot[TALOS_MAX_RANKS];             // this exchange's slot of every rank (rank order)
  unsigned long long* peer_flags[TALOS_MAX_RANKS];
  int world, rank; unsigned long long seq; unsigned spins; int skip_signal;
  int32_t* status;
  float *params, *m, *v, *w_hi, *w_lo, *grads_out, *stats_out;
  long long n;                                    // parameters (a multiple of 4); the slot holds n + 4 floats
  float lr, b1, b2, eps, inv_bc1, inv_bc2;
};
// Launches the fused exchange on the ctx stream (defined in exchange.cu).
void talos_xchg_adam_launch(talos_ctx* ctx, const XchgAdamArgs& a);
