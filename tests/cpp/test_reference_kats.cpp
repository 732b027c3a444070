// The reference crate's own unit tests for this path, replayed through the C++ host mirror
// (talos::Tensor / Module over the C ABI) on the GPU.  Each test names the Rust test it mirrors.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "../../talos-xii_b200/host/talos.hpp"

using namespace talos;
static int failures = 0;
#define EXPECT(cond) do { if (!(cond)) { std::printf("    EXPECT failed: %s (line %d)\n", #cond, __LINE__); ++failures; } } while (0)
#define EXPECT_PANIC(expr) do { bool p_ = false; try { (void)(expr); } catch (const Panic&) { p_ = true; } if (!p_) { std::printf("    expected a panic: %s (line %d)\n", #expr, __LINE__); ++failures; } } while (0)
static void run(const char* name, const std::function<void()>& f) {
  int before = failures;
  try { f(); } catch (const std::exception& e) { std::printf("    exception: %s\n", e.what()); ++failures; }
  std::printf("%s %s\n", failures == before ? "[ OK ]" : "[FAIL]", name);
}
static bool any_abs_gt(const std::vector<double>& v, double t) { for (double x : v) if (std::fabs(x) > t) return true; return false; }

int main(int argc, char** argv) {
  if (argc > 1) Runtime::get().mode = std::stoi(argv[1]);
  std::printf("mode %d\n", Runtime::get().mode);

  run("grad_check::test_autograd_memory_leak_fix", [] {                  // src/grad_check.rs:6-27
    Tensor a = Tensor::new_({2.0}, {1});
    Tensor b = a;
    for (int i = 0; i < 100; ++i) b = b * Tensor::new_({1.1}, {1});
    EXPECT(b._ctx != nullptr);
    Tensor c = b.detach(); EXPECT(c._ctx == nullptr);
    Tensor d = b; d.clear_graph(); EXPECT(d._ctx == nullptr);
    EXPECT(std::fabs(b.item() - 2.0 * std::pow(1.1, 100)) / b.item() < 1e-4);
  });
  run("grad_check::test_grad_check_matmul", [] {                         // src/grad_check.rs:30-63
    Tensor a = Tensor::new_({2.0, 3.0, 4.0, 5.0}, {2, 2}), x = Tensor::new_({1.0, 2.0}, {2, 1});
    Tensor y = a.matmul(x); Tensor loss = y.sum(); loss.backward();
    auto yv = y.to_vec(); EXPECT(yv[0] == 8.0 && yv[1] == 14.0);
    auto ag = a.grad_vec(), xg = x.grad_vec();
    EXPECT(std::fabs(xg[0] - 6.0) < 1e-6 && std::fabs(xg[1] - 8.0) < 1e-6);
    EXPECT(std::fabs(ag[0] - 1.0) < 1e-6 && std::fabs(ag[1] - 2.0) < 1e-6 && std::fabs(ag[2] - 1.0) < 1e-6 && std::fabs(ag[3] - 2.0) < 1e-6);
  });
  run("grad_check::test_grad_check_broadcast", [] {                      // src/grad_check.rs:66-90
    Tensor x = Tensor::new_({1.0, 2.0}, {2}), y = Tensor::new_({10.0}, {1});
    Tensor z = x + y.broadcast({2}); z.sum().backward();
    auto zv = z.to_vec(); EXPECT(zv[0] == 11.0 && zv[1] == 12.0);
    auto xg = x.grad_vec(); EXPECT(std::fabs(xg[0] - 1.0) < 1e-6 && std::fabs(xg[1] - 1.0) < 1e-6);
    EXPECT(std::fabs(y.grad_vec()[0] - 2.0) < 1e-6);
  });
  run("grad_check::test_numerical_gradient_check", [] {                  // src/grad_check.rs:93-114
    const double xv = 2.0, eps = 1e-6;
    Tensor x = Tensor::new_({xv}, {1});
    Tensor y = (x * x) * x.sin(); y.backward();
    auto f = [](double v) { return v * v * std::sin(v); };
    EXPECT(std::fabs(x.grad_vec()[0] - (f(xv + eps) - f(xv - eps)) / (2 * eps)) < 1e-4);
  });
  run("autograd::test_broadcast_scalar", [] {                            // src/autograd.rs:1869-1875
    Tensor b = Tensor::new_({5.0}, {1}).broadcast({2, 2});
    EXPECT((b.shape == std::vector<size_t>{2, 2}));
    for (double v : b.to_vec()) EXPECT(v == 5.0);
  });
  run("autograd: shape errors panic", [] {                               // src/autograd.rs:96-100, :209, :1611
    bool a = false, b = false, c = false;
    try { Tensor::new_({1.0, 2.0}, {3}); } catch (const Panic&) { a = true; }
    try { Tensor::zeros({2, 3}).matmul(Tensor::zeros({4, 2})); } catch (const Panic& e) { b = std::string(e.what()).find("MatMul dimension mismatch") != std::string::npos; }
    try { Tensor::zeros({2}) + Tensor::zeros({3}); } catch (const Panic& e) { c = std::string(e.what()).find("Add shape mismatch") != std::string::npos; }
    EXPECT(a && b && c);
  });
  run("transformer::test_tensor_reshape", [] {                           // src/transformer.rs:1192-1209: reshape is a copy
    Tensor t = Tensor::new_({1.0, 2.0, 3.0, 4.0}, {2, 2});
    Tensor r = t.reshape({4});
    EXPECT((r.shape == std::vector<size_t>{4}) && r.to_vec()[0] == 1.0);
    t.set_data({10.0, 2.0, 3.0, 4.0});
    EXPECT(r.to_vec()[0] == 1.0);
  });
  run("transformer::test_tensor_transpose", [] {                         // src/transformer.rs:1212-1225
    Tensor tt = Tensor::new_({1, 2, 3, 4, 5, 6}, {2, 3}).transpose(0, 1);
    EXPECT((tt.shape == std::vector<size_t>{3, 2}));
    EXPECT((tt.to_vec() == std::vector<double>{1, 4, 2, 5, 3, 6}));
  });
  run("transformer::test_mla_forward_backward", [] {                     // src/transformer.rs:1228-1266
    MultiHeadLatentAttention mla(MLAConfig{16, 2, 0, 8, 4, 8, 10}, 42);
    Tensor input = Tensor::rand({1, 3, 16}, -0.1, 0.1, 123);
    Tensor out = mla.forward(input);
    EXPECT((out.shape == std::vector<size_t>{1, 3, 16}));
    out.mean().backward();
    double s1 = 0, s2 = 0; for (double g : mla.w_dkv.weight.grad_vec()) s1 += g; for (double g : mla.w_uk.weight.grad_vec()) s2 += g;
    EXPECT(std::fabs(s1) > 0.0 && std::fabs(s2) > 0.0);
  });
  run("transformer::test_rope_backward", [] {                            // src/transformer.rs:1269-1281
    RoPE rope(4, 10);
    Tensor x = Tensor::rand({1, 2, 4}, -1.0, 1.0, 123);
    rope.forward(x, 0).sum().backward();
    EXPECT(any_abs_gt(x.grad_vec(), 1e-6));
  });
  run("transformer::test_rmsnorm_backward", [] {                         // src/transformer.rs:1284-1299
    RMSNorm norm(4, 1e-5, 123);
    Tensor x = Tensor::rand({2, 4}, 0.1, 1.0, 123);
    norm.forward(x).sum().backward();
    EXPECT(any_abs_gt(x.grad_vec(), 1e-6) && any_abs_gt(norm.weight.grad_vec(), 1e-6));
  });
  run("transformer::test_luck_transformer_integration", [] {             // src/transformer.rs:1302-1328
    LuckTransformer t(8, 8, true, 42);
    Tensor x = Tensor::rand({1, 5, 8}, -0.1, 0.1, 123);
    t.forward(x).mean().backward();
    EXPECT(t.parameters().size() > 10);
    EXPECT(any_abs_gt(t.embed.weight.grad_vec(), 0.0) && any_abs_gt(t.norm_1.weight.grad_vec(), 0.0));
  });
  run("ppo::test_actor_critic_shapes", [] {                              // src/ppo.rs:1074-1093
    ActorCritic policy(42);
    Tensor s1 = Tensor::new_(std::vector<double>(8, 0.5), {8});
    EXPECT(policy.forward_actor(s1).shape == std::vector<size_t>{5} && policy.forward_critic(s1).shape == std::vector<size_t>{1});
    Tensor s2 = Tensor::new_(std::vector<double>(40, 0.5), {5, 8});
    EXPECT(policy.forward_actor(s2).shape == std::vector<size_t>{5} && policy.forward_critic(s2).shape == std::vector<size_t>{1});
    Tensor s3 = Tensor::new_(std::vector<double>(40, 0.5), {1, 5, 8});
    EXPECT(policy.forward_actor(s3).shape == std::vector<size_t>{5} && policy.forward_critic(s3).shape == std::vector<size_t>{1});
  });
  run("ppo: last_token cuts the graph", [] {                             // src/transformer.rs:92-109: only the heads receive gradients
    ActorCritic policy(7);
    Tensor s = Tensor::rand({4, 8}, -0.5, 0.5, 3);
    policy.forward_actor(s).sum().backward();
    EXPECT(any_abs_gt(policy.actor_head.weight.grad_vec(), 0.0));
    EXPECT(!any_abs_gt(policy.backbone.embed.weight.grad_vec(), 0.0));
  });
  run("sim::ppo_fast_slow_alignment_distribution", [] {                  // src/sim.rs:1181-1216
    ActorCritic policy(12345);
    const size_t seq = 6, dim = 8;
    std::vector<double> flat(seq * dim);
    for (size_t t = 0; t < seq; ++t) for (size_t i = 0; i < dim; ++i) flat[t * dim + i] = t * 0.01 + i * 0.001;
    auto softmax = [](const std::vector<double>& l) { double mx = -1e300, s = 0; for (double v : l) mx = std::max(mx, v);
      std::vector<double> o(l.size()); for (size_t i = 0; i < l.size(); ++i) { o[i] = std::exp(l[i] - mx); s += o[i]; } for (double& v : o) v /= s; return o; };
    auto slow = softmax(policy.forward_actor(Tensor::new_(flat, {seq, dim})).to_vec());
    KVCache kv(policy.backbone.mla_layer.config.num_heads); kv.clear();
    std::vector<double> last;
    for (size_t t = 0; t < seq; ++t) last = policy.backbone.forward_inference_step(std::vector<double>(flat.begin() + t * dim, flat.begin() + (t + 1) * dim), kv, t);
    auto fast = softmax(policy.actor_head.forward_inference(last));
    double diff = 0; for (size_t i = 0; i < 5; ++i) diff += std::fabs(slow[i] - fast[i]);
    EXPECT(diff < 1e-6);
    policy.backbone.mla_layer.prune_kv_cache(kv, 4); EXPECT(kv.len == 4);           // sliding window, src/transformer.rs:843-874
  });
  run("transformer: graph-free whole-sequence forward_inference equals the tape path with token positions", [] {   // src/transformer.rs:111-150, :562-685
    LuckTransformer t(8, 64, true, 99);
    const size_t seq = 5;
    Tensor x = Tensor::rand({1, seq, 8}, -0.5, 0.5, 17);
    t.mla_layer.token_positions = true;                                   // the graph-free paths rotate by TOKEN position (:583-610)
    const std::vector<double> tape = t.forward(x).to_vec(), flat = t.forward_inference(x.to_vec());
    EXPECT(tape.size() == flat.size() && flat.size() == seq * 64);
    double worst = 0; for (size_t i = 0; i < tape.size(); ++i) worst = std::max(worst, std::fabs(tape[i] - flat[i]));
    EXPECT(worst < (mode() == TALOS_MODE_TF32 ? 5e-3 : 1e-5));           // two routes through the same arithmetic mode
    EXPECT(t.last_token_inference(flat) == std::vector<double>(flat.end() - 64, flat.end()));
  });
  run("ppo: advantage block (reward normalisation, GAE, advantage normalisation)", [] {   // src/ppo.rs:444-480, :650-675
    RunningMeanStd rn; for (double r : {1.0, 2.0, -1.0}) rn.update(r);
    EXPECT(std::fabs(rn.count - 3.0001) < 1e-12);
    const std::vector<double> r{1.0, 2.0, -1.0, 0.5}, v{0.5, 0.25, 0.125, -0.25}; const std::vector<int32_t> term{0, 1, 0, 0};
    // the same arithmetic in f64, written out
    std::vector<double> adv(4), ret(4); double last = 0.0;
    for (int t = 3; t >= 0; --t) {
      const double nr = std::min(10.0, std::max(-10.0, rn.normalize(r[t]))), nt = term[t] ? 0.0 : 1.0, vn = t < 3 ? v[t + 1] : 0.0;
      const double gae = nr + 0.99 * vn * nt - v[t] + 0.99 * 0.95 * nt * last;
      adv[t] = gae; ret[t] = gae + v[t]; last = gae;
    }
    double m = 0; for (double a : adv) m += a; m /= 4; double sd = 0; for (double a : adv) sd += (a - m) * (a - m); sd = std::sqrt(sd / 4) + 1e-8;
    auto got = gae_advantages(Tensor::new_(r, {4}), Tensor::new_(v, {4}), term, rn);
    const std::vector<double> ga = got.first.to_vec(), gr = got.second.to_vec();
    for (int t = 0; t < 4; ++t) { EXPECT(std::fabs(ga[t] - (adv[t] - m) / sd) < 1e-5); EXPECT(std::fabs(gr[t] - ret[t]) < 1e-5); }
  });
  run("autograd: save_binary / from_mmap and the serde-bincode tensor layout", [] {   // src/autograd.rs:22-92
    Tensor t = Tensor::new_({1.0, -2.5, 3.25, 4.0, 0.5, -6.0}, {2, 3});
    const std::string path = "/tmp/talos_tensor_io_test.bin";
    EXPECT(t.save_binary(path));
    Tensor back = Tensor::from_mmap(path, {3, 2});                              // the reader supplies the shape
    EXPECT(back.to_vec() == t.to_vec() && back.shape == std::vector<size_t>({3, 2}));
    EXPECT_PANIC(Tensor::from_mmap(path, {7}));                                 // "Mmap size mismatch"
    std::remove(path.c_str());
    const std::vector<uint8_t> b = t.to_bincode();
    EXPECT(b.size() == 8 + 6 * 8 + 8 + 2 * 8);
    const uint8_t head[8] = {6, 0, 0, 0, 0, 0, 0, 0}; EXPECT(std::memcmp(b.data(), head, 8) == 0);      // u64 LE element count
    double first; std::memcpy(&first, b.data() + 8, 8); EXPECT(first == 1.0);
    const uint8_t rank[8] = {2, 0, 0, 0, 0, 0, 0, 0}; EXPECT(std::memcmp(b.data() + 56, rank, 8) == 0);
    std::vector<uint8_t> two = b; two.insert(two.end(), b.begin(), b.end());    // two tensors back to back, as inside Linear
    size_t off = 0; Tensor a1 = Tensor::from_bincode(two, &off), a2 = Tensor::from_bincode(two, &off);
    EXPECT(off == two.size() && a1.to_vec() == t.to_vec() && a2.shape == t.shape);
    two.pop_back(); off = 0; Tensor::from_bincode(two, &off); EXPECT_PANIC(Tensor::from_bincode(two, &off));   // truncated second record
  });
  run("dqn: DuelingQNetwork mirror, double-DQN loss, soft update", [] {     // src/dqn.rs:46-160, :482-584
    DuelingQNetwork policy(7), target(7);
    Tensor states = Tensor::rand({64, 8}, -1.0, 1.0, 9), next = Tensor::rand({64, 8}, -1.0, 1.0, 11);
    // the fused combination equals the crate's three-matmul spelling
    Tensor x = policy.l2.forward(policy.l1.forward(states).relu()).relu();
    Tensor v = policy.val_head.forward(x), a = policy.adv_head.forward(x);
    Tensor ones15 = Tensor::new_(std::vector<double>(5, 1.0), {1, 5}), fifth = Tensor::new_(std::vector<double>(5, 0.2), {5, 1});
    const std::vector<double> spelled = (v.matmul(ones15) + a - a.matmul(fifth).matmul(ones15)).to_vec(), fused = policy.forward(states).to_vec();
    double worst = 0; for (size_t i = 0; i < fused.size(); ++i) worst = std::max(worst, std::fabs(fused[i] - spelled[i]));
    EXPECT(worst < 1e-5);
    EXPECT(policy.forward(Tensor::rand({8}, -1.0, 1.0, 3)).shape == std::vector<size_t>({5}));    // single-state branch
    std::vector<int32_t> actions(64); std::vector<double> rewards(64), dones(64);
    for (int i = 0; i < 64; ++i) { actions[i] = i % 5; rewards[i] = 0.1 * (i % 7) - 0.3; dones[i] = (i % 9 == 0) ? 1.0 : 0.0; }
    std::vector<Tensor> params = policy.parameters();
    Adam opt(params, 1e-3); opt.clip_norm = 1.0;                                                 // src/dqn.rs:207-239
    double first = 0, last = 0;
    for (int it = 0; it < 40; ++it) {
      opt.zero_grad();
      Tensor loss = dqn_loss(policy.forward(states), actions, policy.forward(next), target.forward(next), rewards, dones);
      loss.backward(); opt.step();
      target.soft_update(policy, 0.005);
      if (it == 0) first = loss.item();
      last = loss.item();
    }
    EXPECT(std::isfinite(last) && last < first);
    // (with the crate's half-range LCG every weight is negative, so the second ReLU layer is dead and only the head
    //  biases learn: they are what the soft update has to track)
    const std::vector<double> tw = target.val_head.bias->to_vec(), pw = policy.val_head.bias->to_vec();
    double moved = 0, gap = 0; DuelingQNetwork fresh(7); const std::vector<double> fw = fresh.val_head.bias->to_vec();
    for (size_t i = 0; i < tw.size(); ++i) { moved += std::fabs(tw[i] - fw[i]); gap += std::fabs(tw[i] - pw[i]); }
    EXPECT(moved > 0 && gap > 0);                                                                // the target trails the policy
    target.load_state_dict(policy); EXPECT(target.l2.weight.to_vec() == policy.l2.weight.to_vec());
    EXPECT(policy.predict_action(Tensor::rand({8}, -1.0, 1.0, 5)) < 5);
  });
  run("dqn: dueling network consumer (batch 64) trains", [] {            // src/dqn.rs:68-107, :207-239, :482-584
    Linear l1(8, 64, true, 1), l2(64, 64, true, 2), val(64, 1, true, 3), adv(64, 5, true, 4);
    auto fwd = [&](const Tensor& s) {
      Tensor x = l2.forward(l1.forward(s).relu()).relu();
      Tensor v = val.forward(x), a = adv.forward(x);
      Tensor ones15 = Tensor::new_(std::vector<double>(5, 1.0), {1, 5}), fifth = Tensor::new_(std::vector<double>(5, 0.2), {5, 1});
      return v.matmul(ones15) + a - a.matmul(fifth).matmul(ones15);                  // Q = V + A - mean(A)
    };
    std::vector<Tensor> params; for (Linear* l : {&l1, &l2, &val, &adv}) for (auto& p : l->parameters()) params.push_back(p);
    Adam opt(params, 1e-3); opt.clip_norm = 1.0;
    Tensor states = Tensor::rand({64, 8}, -1.0, 1.0, 9), target = Tensor::rand({64, 5}, -1.0, 1.0, 10);
    double first = 0, last = 0;
    for (int it = 0; it < 30; ++it) {
      opt.zero_grad();
      Tensor loss = fwd(states).mse_loss(target);
      loss.backward(); opt.step();
      if (it == 0) first = loss.item();
      last = loss.item();
    }
    EXPECT(last < first && std::isfinite(last));
  });
  std::printf("%d failure(s)\n", failures);
  return failures ? 1 : 0;
}
