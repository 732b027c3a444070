// Runs a reference-sized model through the C++ host mirror and dumps the results as raw f64 for the
// Python parity tests to compare with the oracle.  Usage: host_driver <scenario> <mode> <out.bin> [args]
//   luck  <seed> <B> <S> <in> <hidden> : LuckTransformer forward on LCG input, loss = mean, backward;
//                                        writes output, x.grad, then every parameter's grad in parameters() order.
//   mla   <seed> <B> <S>               : MultiHeadLatentAttention (dim16/h2/r8/rope4/dv8) forward/backward, same layout.
//   block <dumpB> <B> 0 [start]        : benchmark config 3 (S64 d256 H8 ff1024, N(0,0.02^2) weights seeds 11-14, x seed 10,
//                                        upstream gradient seed 15); loss = sum(out*G); writes fp32: out, dx (dumpB samples
//                                        each, beginning at sample `start`), then the six parameter gradients.
//   mla4  <dumpB> <B> <token> [start]  : benchmark config 4 (S128 d512 r64 H8 dh64 dr32, seeds 20-27) forward; writes fp32 out
//                                        of dumpB samples beginning at sample `start`.
//   serde <seed> <B> <S> <prefix>      : ActorCritic(seed) written with save_ppo_model to <prefix>.bin (bincode) and <prefix>
//                                        (JSON), read back from each and through load_ppo_model (binary first; JSON when
//                                        only <prefix>.json_only exists); writes f64 actor logits on LCG states [B,S,8] of the
//                                        original and of the four loaded models, [5][B,5].
//   time  <seed> <iters> <batch>       : no dump; times the two training routes that go through the Tensor tape -- a dueling
//                                        double-DQN train step at batch `batch` (forward x3, loss, backward, clipped Adam, soft
//                                        update: src/dqn.rs:482-584) and a LuckTransformer(8, 64) forward + backward on
//                                        [batch, 16, 8] -- and prints one JSON line with steps per second and the allocator's counters.
//   rollout <seed> <N> <T> <ctx> [time]: ActorCritic(seed) stepped T times over N simulations through BatchedRollout
//                                        (KV rings of ctx+1 slots); states N(0, 0.5^2) seed+500 as [T,N,8]; simulation n
//                                        ends an episode after step t when (t*7 + n*3) % 11 == 0; writes f64 probabilities
//                                        [T,N,5].  With `time`: no dump, prints simulation-steps per second instead.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "../../talos-xii_b200/host/talos_serde.hpp"
using namespace talos;

static void dump(std::FILE* f, const std::vector<double>& v) { std::fwrite(v.data(), sizeof(double), v.size(), f); }
static void dump32(std::FILE* f, const std::vector<double>& v, size_t count, size_t first = 0) {
  std::vector<float> t(count); for (size_t i = 0; i < count; ++i) t[i] = (float)v[first + i]; std::fwrite(t.data(), sizeof(float), count, f);
}
static Tensor normal(std::vector<size_t> shape, uint64_t seed, float std_dev) {
  std::vector<float> h(numel(shape)); check(talos_rng_normal_host(seed, 0.f, std_dev, h.data(), (int64_t)h.size()));
  return Tensor::new_(std::vector<double>(h.begin(), h.end()), std::move(shape));
}
static void set_normal(Linear& l, uint64_t seed) { l.weight = normal({l.in_features, l.out_features}, seed, 0.02f); }
// The crate's LCG fills [-limit, 0) only; w <- 2w + limit spreads the same stream over [-limit, limit) so
// that the softmax is not saturated and every gradient is well conditioned.
static void symmetrise(Linear& l) {
  const double limit = std::sqrt(6.0 / (double)(l.in_features + l.out_features));
  std::vector<double> w = l.weight.to_vec(); for (double& v : w) v = 2.0 * v + limit; l.weight.set_data(w);
}

int main(int argc, char** argv) {
  if (argc < 4) { std::fprintf(stderr, "usage\n"); return 2; }
  try {
    std::string what = argv[1]; Runtime::get().mode = std::stoi(argv[2]);
    std::FILE* f = std::fopen(argv[3], "wb"); if (!f) return 3;
    uint64_t seed = std::stoull(argv[4]); size_t B = std::stoul(argv[5]), S = std::stoul(argv[6]);
    const bool sym = std::getenv("TALOS_SYMMETRIC_WEIGHTS") != nullptr;
    if (what == "luck") {
      size_t in = std::stoul(argv[7]), hidden = std::stoul(argv[8]);
      LuckTransformer t(in, hidden, true, seed);
      if (sym) { for (Linear* l : {&t.embed, &t.ffn_1, &t.ffn_2, &t.out_proj, &t.mla_layer.w_dkv, &t.mla_layer.w_uk, &t.mla_layer.w_uv, &t.mla_layer.w_q,
                                   &t.mla_layer.w_kr, &t.mla_layer.w_qr, &t.mla_layer.w_o}) symmetrise(*l); }
      Tensor x = Tensor::rand({B, S, in}, -0.5, 0.5, seed + 1000);
      Tensor out = t.forward(x); out.mean().backward();
      dump(f, out.to_vec()); dump(f, x.grad_vec());
      for (auto& p : t.parameters()) dump(f, p.grad_vec());
    } else if (what == "mla") {
      MultiHeadLatentAttention m(MLAConfig{16, 2, 0, 8, 4, 8, 64}, seed);
      if (sym) { for (Linear* l : {&m.w_dkv, &m.w_uk, &m.w_uv, &m.w_q, &m.w_kr, &m.w_qr, &m.w_o}) symmetrise(*l); }
      Tensor x = Tensor::rand({B, S, 16}, -0.5, 0.5, seed + 1000);
      Tensor out = m.forward(x); out.mean().backward();
      dump(f, out.to_vec()); dump(f, x.grad_vec());
      for (auto& p : m.parameters()) dump(f, p.grad_vec());
    } else if (what == "block") {
      const size_t dumpB = seed, Bn = B, Sq = 64, D = 256, start = argc > 7 ? std::stoul(argv[7]) : 0;
      TransformerBlock blk(D, 8, 1024, Sq, 1e-6, 0);
      set_normal(blk.w_qkv, 11); set_normal(blk.w_o, 12); set_normal(blk.w_ff1, 13); set_normal(blk.w_ff2, 14);
      Tensor x = normal({Bn, Sq, D}, 10, 1.f), G = normal({Bn, Sq, D}, 15, 1.f);
      Tensor out = blk.forward(x); (out * G).sum().backward();
      dump32(f, out.to_vec(), dumpB * Sq * D, start * Sq * D); dump32(f, x.grad_vec(), dumpB * Sq * D, start * Sq * D);
      for (auto& p : blk.parameters()) dump32(f, p.grad_vec(), p.len());
    } else if (what == "mla4") {
      const size_t dumpB = seed, Bn = B, Sq = 128, D = 512, start = argc > 7 ? std::stoul(argv[7]) : 0;
      MultiHeadLatentAttention m(MLAConfig{D, 8, 0, 64, 32, 64, 128}, 0);
      m.token_positions = S != 0;
      set_normal(m.w_dkv, 21); set_normal(m.w_uk, 22); set_normal(m.w_uv, 23); set_normal(m.w_q, 24); set_normal(m.w_kr, 25); set_normal(m.w_qr, 26); set_normal(m.w_o, 27);
      Tensor x = normal({Bn, Sq, D}, 20, 1.f);
      Tensor out = m.forward(x);
      dump32(f, out.to_vec(), dumpB * Sq * D, start * Sq * D);
    } else if (what == "serde") {
      const std::string prefix = argv[7];
      ActorCritic ac(seed);
      if (!serde::save_ppo_model(ac, prefix)) { std::fprintf(stderr, "host_driver: cannot write %s\n", prefix.c_str()); return 6; }
      std::string raw, js;
      if (!serde::read_file(prefix + ".bin", &raw) || !serde::read_file(prefix, &js)) return 6;
      ActorCritic from_bin = serde::actor_critic_from_bincode(std::vector<uint8_t>(raw.begin(), raw.end()));
      ActorCritic from_json = serde::actor_critic_from_json(js);
      std::optional<ActorCritic> loaded = serde::load_ppo_model(prefix);                       // finds the binary file
      if (!serde::write_file(prefix + ".json_only", js.data(), js.size())) return 6;
      std::optional<ActorCritic> loaded_json = serde::load_ppo_model(prefix + ".json_only");  // no .bin beside it: JSON
      if (!loaded || !loaded_json || serde::load_ppo_model(prefix + ".missing")) { std::fprintf(stderr, "host_driver: load_ppo_model\n"); return 7; }
      Tensor x = Tensor::rand({B, S, ActorCritic::DIM}, -0.5, 0.5, seed + 1000);
      for (const ActorCritic* m : {&ac, &from_bin, &from_json, &*loaded, &*loaded_json}) dump(f, m->forward_actor(x).to_vec());
      // a second save of a loaded model must reproduce the files byte for byte
      if (serde::to_bincode(from_json) != std::vector<uint8_t>(raw.begin(), raw.end()) || serde::to_json(from_bin) != js) { std::fprintf(stderr, "host_driver: re-serialised model differs\n"); return 8; }
    } else if (what == "time") {
      const size_t iters = B, batch = S;
      DuelingQNetwork policy(seed), target(seed);
      Tensor states = Tensor::rand({batch, 8}, -1.0, 1.0, seed + 1), next = Tensor::rand({batch, 8}, -1.0, 1.0, seed + 2);
      std::vector<int32_t> actions(batch); std::vector<double> rewards(batch), dones(batch);
      for (size_t i = 0; i < batch; ++i) { actions[i] = (int32_t)(i % 5); rewards[i] = 0.1 * (double)(i % 7) - 0.3; dones[i] = (i % 9 == 0) ? 1.0 : 0.0; }
      Adam opt(policy.parameters(), 1e-3); opt.clip_norm = 1.0;
      auto dqn_step = [&]() {
        opt.zero_grad();
        Tensor loss = dqn_loss(policy.forward(states), actions, policy.forward(next), target.forward(next), rewards, dones);
        loss.backward(); opt.step(); target.soft_update(policy, 0.005);
      };
      auto timed = [&](auto&& fn) {
        for (int i = 0; i < 3; ++i) fn();
        Runtime::get().synchronize();
        const auto t0 = std::chrono::steady_clock::now();
        for (size_t i = 0; i < iters; ++i) fn();
        Runtime::get().synchronize();
        return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() / (double)iters;
      };
      int64_t st0[4], st1[4];
      const double dqn_s = timed(dqn_step);
      LuckTransformer lt(8, 64, true, seed); Tensor x = Tensor::rand({batch, 16, 8}, -0.5, 0.5, seed + 3);
      auto params = lt.parameters();
      auto luck_step = [&]() { for (auto& p : params) p.zero_grad(); lt.forward(x).mean().backward(); };
      luck_step(); Runtime::get().synchronize();
      check(talos_ctx_memory_stats(ctx(), st0));
      const double luck_s = timed(luck_step);
      check(talos_ctx_memory_stats(ctx(), st1));
      std::printf("{\"dqn_train_step_ms\": %.4f, \"dqn_steps_per_s\": %.1f, \"luck_fwd_bwd_ms\": %.4f, \"batch\": %zu, \"iters\": %zu, "
                  "\"luck_driver_allocations_while_timed\": %lld, \"luck_allocations_from_cache_while_timed\": %lld, \"cached_bytes\": %lld}\n",
                  dqn_s * 1e3, 1.0 / dqn_s, luck_s * 1e3, batch, iters, (long long)(st1[2] - st0[2]), (long long)(st1[3] - st0[3]), (long long)st1[1]);
    } else if (what == "rollout") {
      const size_t N = B, T = S, ctx_len = std::stoul(argv[7]);
      const bool timing = argc > 8 && std::string(argv[8]) == "time";
      ActorCritic ac(seed);
      if (sym) {
        LuckTransformer& t = ac.backbone;
        for (Linear* l : {&t.embed, &t.ffn_1, &t.ffn_2, &t.out_proj, &t.mla_layer.w_dkv, &t.mla_layer.w_uk, &t.mla_layer.w_uv, &t.mla_layer.w_q,
                          &t.mla_layer.w_kr, &t.mla_layer.w_qr, &t.mla_layer.w_o, &ac.actor_head}) symmetrise(*l);
      }
      BatchedRollout roll(ac, N, ctx_len);
      if (!timing) {
        Tensor states = normal({T, N, ActorCritic::DIM}, seed + 500, 0.5f);
        const std::vector<double> sv = states.to_vec();
        for (size_t t = 0; t < T; ++t) {
          std::vector<int32_t> reset(N);
          for (size_t n = 0; n < N; ++n) reset[n] = ((t * 7 + n * 3) % 11 == 0) ? 1 : 0;
          std::vector<double> st(sv.begin() + t * N * ActorCritic::DIM, sv.begin() + (t + 1) * N * ActorCritic::DIM);
          dump(f, roll.step_host(st, &reset));
        }
      } else {
        Tensor states = normal({N, ActorCritic::DIM}, seed + 500, 0.5f);
        for (size_t t = 0; t < 3; ++t) roll.step(states.d());
        Runtime::get().synchronize();
        const auto t0 = std::chrono::steady_clock::now();          // host clock between two stream synchronisations
        for (size_t t = 0; t < T; ++t) roll.step(states.d());
        Runtime::get().synchronize();
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        std::printf("{\"kernel\": \"batched_rollout_step\", \"sims\": %zu, \"context_len\": %zu, \"steps\": %zu, \"ms_per_step\": %.4f, \"sim_steps_per_s\": %.1f}\n",
                    N, ctx_len, T, ms / T, (double)N * T / (ms * 1e-3));
      }
    } else { return 4; }
    std::fclose(f);
    // a failed tensor-core self-check must fail the run, not hide behind the fp32 stand-in
    if (Runtime::get().mode != TALOS_MODE_FP32 && talos_ctx_tensor_cores_state(ctx()) < 0) { std::fprintf(stderr, "host_driver: tensor-core self-check failed\n"); return 5; }
  } catch (const std::exception& e) { std::fprintf(stderr, "host_driver: %s\n", e.what()); return 1; }
  return 0;
}
