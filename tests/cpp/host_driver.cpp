// Runs a reference-sized model through the C++ host mirror and dumps the results as raw f64 for the
// Python parity tests to compare with the oracle.  Usage: host_driver <scenario> <mode> <out.bin> [args]
//   luck  <seed> <B> <S> <in> <hidden> : LuckTransformer forward on LCG input, loss = mean, backward;
//                                        writes output, x.grad, then every parameter's grad in parameters() order.
//   mla   <seed> <B> <S>               : MultiHeadLatentAttention (dim16/h2/r8/rope4/dv8) forward/backward, same layout.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "../../talos-xii_b200/host/talos.hpp"
using namespace talos;

static void dump(std::FILE* f, const std::vector<double>& v) { std::fwrite(v.data(), sizeof(double), v.size(), f); }
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
    } else { return 4; }
    std::fclose(f);
  } catch (const std::exception& e) { std::fprintf(stderr, "host_driver: %s\n", e.what()); return 1; }
  return 0;
}
