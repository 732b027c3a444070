// C++ host mirror of the reference crate's Tensor / autograd / Module API on top of the talos_b200 C ABI.
//
// The reference's host language is Rust; this header plays the role its `ffi.rs` + thin wrapper types
// would play: same type and method names, same argument meaning, same error behaviour (a shape
// mismatch the crate reports with assert!/panic! is thrown here as talos::Panic).  It binds nothing but
// include/talos_b200.h -- no CUDA runtime -- exactly like a foreign-language host would.
//
//   Tensor          src/autograd.rs:15-196, ops :200-792, operators :1608-1862
//   Module, Linear  src/nn.rs:6-142          RMSNorm  src/nn.rs:145-304
//   RoPE, MLAConfig, MultiHeadLatentAttention, KVCache, LuckTransformer   src/transformer.rs
//   ActorCritic, Adam   src/ppo.rs:247-540   (Adam with clip_norm = 1: src/dqn.rs:207-239)
//
// Device data is fp32; the crate's f64 vectors are converted at to_vec()/from-vector boundaries.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <memory>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/talos_b200.h"

namespace talos {

struct Panic : std::runtime_error { using std::runtime_error::runtime_error; };

inline void check(talos_status st) {
  if (st != TALOS_OK) throw Panic(std::string("talos_b200 status ") + std::to_string(st) + ": " + talos_last_error_string());
}
#define TALOS_ASSERT(cond, msg) do { if (!(cond)) throw talos::Panic(msg); } while (0)

// One device + stream and the GEMM arithmetic used by every op (process-wide, like the crate's global Rayon pool).
class Runtime {
 public:
  static Runtime& get() { static Runtime r; return r; }
  talos_ctx* ctx() { if (!ctx_) check(talos_ctx_create(device_, nullptr, &ctx_)); return ctx_; }
  int mode = TALOS_MODE_TF32X3;
  void set_device(int d) { TALOS_ASSERT(ctx_ == nullptr, "set_device after first use"); device_ = d; }
  void synchronize() { check(talos_ctx_synchronize(ctx())); }
 private:
  talos_ctx* ctx_ = nullptr; int device_ = 0;
};
inline talos_ctx* ctx() { return Runtime::get().ctx(); }
inline int mode() { return Runtime::get().mode; }

// Device buffer with shared ownership: the Arc<RwLock<Vec<f64>>> of the crate (src/autograd.rs:16-17).
struct Storage {
  float* dev = nullptr; size_t n = 0;
  explicit Storage(size_t count, bool zero = true) : n(count) {
    void* p = nullptr; check(talos_malloc(ctx(), sizeof(float) * (n ? n : 1), &p)); dev = (float*)p;
    if (zero) check(talos_memset_zero(ctx(), dev, sizeof(float) * n));
  }
  ~Storage() { if (dev) talos_free(ctx(), dev); }
  Storage(const Storage&) = delete; Storage& operator=(const Storage&) = delete;
};
using Buf = std::shared_ptr<Storage>;
inline Buf make_buf(size_t n, bool zero = true) { return std::make_shared<Storage>(n, zero); }

inline size_t numel(const std::vector<size_t>& s) { size_t n = 1; for (size_t d : s) n *= d; return n; }

class Tensor;
struct Context {                                   // src/autograd.rs:51-54
  std::vector<Tensor> parents;
  std::function<void(const Tensor& out, const std::vector<Tensor>& parents)> backward_op;   // reads out.grad
};

class Tensor {
 public:
  Buf data, grad;
  std::vector<size_t> shape;
  std::shared_ptr<Context> _ctx;                   // keeps the graph alive

  Tensor() = default;
  // Tensor::new (src/autograd.rs:94-107)
  static Tensor new_(const std::vector<double>& values, std::vector<size_t> shape) {
    TALOS_ASSERT(values.size() == numel(shape), "Data length must match shape");
    Tensor t; t.shape = std::move(shape); t.data = make_buf(values.size(), false); t.grad = make_buf(values.size());
    check(talos_upload_f64(ctx(), t.data->dev, values.data(), (int64_t)values.size()));
    return t;
  }
  static Tensor zeros(std::vector<size_t> shape) { Tensor t; t.shape = std::move(shape); t.data = make_buf(numel(t.shape)); t.grad = make_buf(numel(t.shape)); return t; }
  // Tensor::rand: the crate's LCG, half range and all (src/autograd.rs:114-124)
  static Tensor rand(std::vector<size_t> shape, double lo, double hi, uint64_t seed) {
    std::vector<double> v(numel(shape)); check(talos_lcg_rand_host(seed, lo, hi, v.data(), (int64_t)v.size())); return new_(v, std::move(shape));
  }
  // Fresh result tensor of an op: uninitialised data, zero grad, recorded parents.
  static Tensor result(std::vector<size_t> shape, std::vector<Tensor> parents,
                       std::function<void(const Tensor&, const std::vector<Tensor>&)> bwd) {
    Tensor t; t.shape = std::move(shape); t.data = make_buf(numel(t.shape), false); t.grad = make_buf(numel(t.shape));
    t._ctx = std::make_shared<Context>(); t._ctx->parents = std::move(parents); t._ctx->backward_op = std::move(bwd);
    return t;
  }
  size_t len() const { return data ? data->n : 0; }
  float* d() const { return data->dev; }
  float* g() const { return grad->dev; }

  Tensor detach() const { Tensor t = *this; t._ctx = nullptr; return t; }          // shares data and grad (:126-137)
  void clear_graph() { _ctx = nullptr; }                                          // :187-189
  void zero_grad() const { check(talos_memset_zero(ctx(), grad->dev, sizeof(float) * grad->n)); }
  std::vector<double> to_vec() const { std::vector<double> v(len()); check(talos_download_f64(ctx(), v.data(), d(), (int64_t)v.size())); return v; }
  std::vector<double> grad_vec() const { std::vector<double> v(len()); check(talos_download_f64(ctx(), v.data(), g(), (int64_t)v.size())); return v; }
  void set_data(const std::vector<double>& v) const { TALOS_ASSERT(v.size() == len(), "Data length must match shape"); check(talos_upload_f64(ctx(), d(), v.data(), (int64_t)v.size())); }
  // ---- file formats of the crate, so that cached models move between the two implementations ----
  // save_binary / from_mmap (src/autograd.rs:56-92): the data as raw little-endian f64, nothing else; the shape is
  // supplied by the reader, which fails with "Mmap size mismatch" when the byte count does not fit it.
  bool save_binary(const std::string& path) const {
    std::FILE* f = std::fopen(path.c_str(), "wb"); if (!f) return false;
    const std::vector<double> v = to_vec();
    const bool ok = std::fwrite(v.data(), sizeof(double), v.size(), f) == v.size();
    return std::fclose(f) == 0 && ok;
  }
  static Tensor from_mmap(const std::string& path, std::vector<size_t> shape) {
    std::FILE* f = std::fopen(path.c_str(), "rb"); TALOS_ASSERT(f != nullptr, "cannot open tensor file");
    std::vector<double> v(numel(shape) + 1);
    const size_t got = std::fread(v.data(), sizeof(double), v.size(), f); std::fclose(f);
    TALOS_ASSERT(got == numel(shape), "Mmap size mismatch");
    v.resize(numel(shape));
    return new_(v, std::move(shape));
  }
  // The serde layout `struct Tensor { data: Vec<f64>, shape: Vec<usize> }` (src/autograd.rs:22-50) as bincode 1.x
  // writes it with its default options: u64 little-endian element count, the f64 values, u64 rank, u64 dimensions.
  std::vector<uint8_t> to_bincode() const {
    const std::vector<double> v = to_vec();
    std::vector<uint8_t> out(8 + 8 * v.size() + 8 + 8 * shape.size());
    uint8_t* p = out.data();
    auto put = [&p](uint64_t x) { std::memcpy(p, &x, 8); p += 8; };
    put(v.size()); std::memcpy(p, v.data(), 8 * v.size()); p += 8 * v.size();
    put(shape.size()); for (size_t d : shape) put((uint64_t)d);
    return out;
  }
  // Reads one tensor starting at bytes[*offset]; advances *offset past it (tensors are simply concatenated inside
  // the structs that hold them).  Panics on a truncated buffer or a shape that does not match the data length.
  static Tensor from_bincode(const std::vector<uint8_t>& bytes, size_t* offset) {
    size_t o = *offset;
    auto get = [&](uint64_t* x) { TALOS_ASSERT(o + 8 <= bytes.size(), "truncated tensor record"); std::memcpy(x, bytes.data() + o, 8); o += 8; };
    uint64_t n = 0, rank = 0; get(&n);
    TALOS_ASSERT(n <= (bytes.size() - o) / 8, "truncated tensor record");
    std::vector<double> v(n); std::memcpy(v.data(), bytes.data() + o, 8 * n); o += 8 * n;
    get(&rank); TALOS_ASSERT(rank <= 8, "tensor rank out of range");
    std::vector<size_t> shp(rank); for (auto& d : shp) { uint64_t x; get(&x); d = (size_t)x; }
    TALOS_ASSERT(numel(shp) == n, "Data length must match shape");
    *offset = o;
    return new_(v, std::move(shp));
  }
  double item() const { TALOS_ASSERT(numel(shape) == 1, "item() needs one element"); return to_vec()[0]; }

  // Tensor::backward (src/autograd.rs:145-184): DFS topological order keyed on the grad buffer, root grad = 1.
  void backward() const {
    std::vector<Tensor> topo; std::set<const Storage*> seen;
    std::function<void(const Tensor&)> visit = [&](const Tensor& t) {
      if (seen.count(t.grad.get())) return;
      seen.insert(t.grad.get());
      if (t._ctx) for (const Tensor& p : t._ctx->parents) visit(p);
      topo.push_back(t);
    };
    visit(*this);
    std::vector<double> ones(len(), 1.0);
    check(talos_upload_f64(ctx(), g(), ones.data(), (int64_t)ones.size()));
    for (auto it = topo.rbegin(); it != topo.rend(); ++it) if (it->_ctx) it->_ctx->backward_op(*it, it->_ctx->parents);
  }

  // ---- ops --------------------------------------------------------------------------------------
  Tensor matmul(const Tensor& other) const {                                       // src/autograd.rs:200-354
    TALOS_ASSERT(shape.size() <= 2 && other.shape.size() == 2, "matmul needs lhs rank <= 2 and rhs rank 2");
    const size_t m = shape.size() == 1 ? 1 : shape[0], k = shape.size() == 1 ? shape[0] : shape[1];
    const size_t k2 = other.shape[0], n = other.shape[1];
    TALOS_ASSERT(k == k2, "MatMul dimension mismatch");
    std::vector<size_t> os = shape.size() == 1 ? std::vector<size_t>{n} : std::vector<size_t>{m, n};
    Tensor out = result(os, {*this, other}, [m, k, n](const Tensor& o, const std::vector<Tensor>& p) {
      talos_epilogue acc{}; acc.beta = 1;                                           // gradients accumulate (:304, :346)
      check(talos_gemm(ctx(), TALOS_OP_N, TALOS_OP_T, m, k, n, o.g(), n, p[1].d(), n, p[0].g(), k, mode(), &acc));   // dLHS = G.B^T
      check(talos_gemm(ctx(), TALOS_OP_T, TALOS_OP_N, k, n, m, p[0].d(), k, o.g(), n, p[1].g(), n, mode(), &acc));   // dRHS = A^T.G
    });
    check(talos_gemm(ctx(), TALOS_OP_N, TALOS_OP_N, m, n, k, d(), k, other.d(), n, out.d(), n, mode(), nullptr));
    return out;
  }
  Tensor unary(int op, float p0 = 0.f, float p1 = 0.f) const {
    Tensor out = result(shape, {*this}, [op, p0, p1](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_eltwise_unary_bwd(ctx(), op, p[0].d(), o.g(), p[0].g(), (int64_t)o.len(), p0, p1));
    });
    check(talos_eltwise_unary(ctx(), op, d(), out.d(), (int64_t)len(), p0, p1));
    return out;
  }
  Tensor relu() const { return unary(TALOS_EW_RELU); }                              // :356-386
  Tensor log() const { return unary(TALOS_EW_LOG); }                                // :388-413
  Tensor exp() const { return unary(TALOS_EW_EXP); }                                // :415-441
  Tensor sin() const { return unary(TALOS_EW_SIN); }                                // :549-574
  Tensor cos() const { return unary(TALOS_EW_COS); }                                // :576-601
  Tensor sqrt() const { return unary(TALOS_EW_SQRT); }                              // :603-630
  Tensor clip(double lo, double hi) const { return unary(TALOS_EW_CLIP, (float)lo, (float)hi); }   // :741-768
  Tensor tanh() const { return unary(TALOS_EW_TANH); }                              // not in the crate
  Tensor silu() const { return unary(TALOS_EW_SILU); }                              // not in the crate
  Tensor scale(double s) const { return unary(TALOS_EW_SCALE, (float)s); }          // scale_tensor, src/transformer.rs:1052-1072
  Tensor reduce(double factor) const {
    const size_t n = len();
    Tensor out = result({1}, {*this}, [factor, n](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_fill_from_scalar(ctx(), o.g(), (float)factor, p[0].g(), (int64_t)n, 1));
    });
    check(talos_reduce_sum(ctx(), d(), (int64_t)n, (float)factor, out.d(), 0));
    return out;
  }
  Tensor sum() const { return reduce(1.0); }                                        // :443-461
  Tensor mean() const { return reduce(1.0 / (double)len()); }                       // :463-482
  Tensor broadcast(std::vector<size_t> new_shape) const {                           // :484-509
    TALOS_ASSERT(shape == std::vector<size_t>{1}, "Broadcast only supported for scalar (1) to N");
    Tensor out = result(new_shape, {*this}, [](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_reduce_sum(ctx(), o.g(), (int64_t)o.len(), 1.f, p[0].g(), 1));
    });
    check(talos_fill_from_scalar(ctx(), d(), 1.f, out.d(), (int64_t)out.len(), 0));
    return out;
  }
  Tensor broadcast_to_batch(size_t batch) const {                                   // :511-547
    std::vector<size_t> ns{batch}; ns.insert(ns.end(), shape.begin(), shape.end());
    const size_t n = len();
    Tensor out = result(ns, {*this}, [batch, n](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_colsum(ctx(), o.g(), p[0].g(), (int64_t)batch, (int64_t)n, 1));
    });
    check(talos_memset_zero(ctx(), out.d(), sizeof(float) * out.len()));
    check(talos_bias_add(ctx(), out.d(), d(), (int64_t)batch, (int64_t)n));
    return out;
  }
  Tensor transpose(size_t d0, size_t d1) const {                                    // :632-739
    TALOS_ASSERT(d0 < shape.size() && d1 < shape.size(), "transpose axis out of range");
    std::vector<size_t> ns = shape; std::swap(ns[d0], ns[d1]);
    std::vector<int64_t> in_shape(shape.begin(), shape.end()), out_shape(ns.begin(), ns.end());
    Tensor out = result(ns, {*this}, [out_shape, d0, d1](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_transpose(ctx(), o.g(), p[0].g(), out_shape.data(), (int32_t)out_shape.size(), (int32_t)d0, (int32_t)d1, 1));
    });
    check(talos_transpose(ctx(), d(), out.d(), in_shape.data(), (int32_t)in_shape.size(), (int32_t)d0, (int32_t)d1, 0));
    return out;
  }
  Tensor reshape(std::vector<size_t> new_shape) const {                             // :770-792 -- a COPY, as in the crate
    TALOS_ASSERT(numel(new_shape) == len(), "Reshape dimension mismatch");
    Tensor out = result(new_shape, {*this}, [](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_eltwise_binary(ctx(), TALOS_EW_ADD, p[0].g(), o.g(), p[0].g(), (int64_t)o.len()));
    });
    check(talos_copy_device(ctx(), out.d(), d(), sizeof(float) * len()));
    return out;
  }
  Tensor binary(int op, const Tensor& rhs, const char* what) const {                // :1608-1831
    TALOS_ASSERT(shape == rhs.shape, std::string(what) + " shape mismatch");
    Tensor out = result(shape, {*this, rhs}, [op](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_eltwise_binary_bwd(ctx(), op, p[0].d(), p[1].d(), o.g(), p[0].g(), p[1].g(), (int64_t)o.len()));   // aliased operands ok (:1729)
    });
    check(talos_eltwise_binary(ctx(), op, d(), rhs.d(), out.d(), (int64_t)len()));
    return out;
  }
  Tensor operator+(const Tensor& r) const { return binary(TALOS_EW_ADD, r, "Add"); }
  Tensor operator-(const Tensor& r) const { return binary(TALOS_EW_SUB, r, "Sub"); }
  Tensor operator*(const Tensor& r) const { return binary(TALOS_EW_MUL, r, "Mul"); }
  Tensor operator/(const Tensor& r) const { return binary(TALOS_EW_DIV, r, "Div"); }
  Tensor operator-() const { return unary(TALOS_EW_NEG); }                          // :1833-1862
  Tensor mse_loss(const Tensor& target) const { Tensor diff = *this - target; return (diff * diff).mean(); }   // :1599-1603
};

// ---- layers -------------------------------------------------------------------------------------
struct Module {                                                                     // src/nn.rs:6-9
  virtual ~Module() = default;
  virtual Tensor forward(const Tensor& input) const = 0;
  virtual std::vector<Tensor> parameters() const = 0;
};

inline size_t rows_of(const Tensor& x, size_t last) { TALOS_ASSERT(!x.shape.empty() && x.shape.back() == last, "MatMul dimension mismatch"); return x.len() / last; }

// Tag for constructing a layer whose fields a deserialiser fills in afterwards (no random initialisation, no upload).
struct Uninit {};

struct Linear : Module {                                                            // src/nn.rs:12-142
  Tensor weight; std::optional<Tensor> bias; size_t in_features, out_features;
  explicit Linear(Uninit) : in_features(0), out_features(0) {}
  Linear(size_t in_f, size_t out_f, bool with_bias, uint64_t seed) : in_features(in_f), out_features(out_f) {
    const double limit = std::sqrt(6.0 / (double)(in_f + out_f));                   // Xavier (:22)
    weight = Tensor::rand({in_f, out_f}, -limit, limit, seed);
    if (with_bias) bias = Tensor::zeros({out_f});
  }
  // y = act(x.W + b) as ONE tape node; the crate builds reshape -> matmul -> reshape -> broadcast -> add (:73-133).
  Tensor forward_act(const Tensor& x, int act) const {
    const size_t rows = rows_of(x, in_features), in_f = in_features, out_f = out_features;
    std::vector<size_t> os = x.shape; os.back() = out_f;
    std::vector<Tensor> parents{x, weight}; if (bias) parents.push_back(*bias);
    Buf saved_z = act == TALOS_ACT_SILU ? make_buf(rows * out_f, false) : nullptr;
    Tensor out = Tensor::result(os, parents, [rows, in_f, out_f, act, saved_z](const Tensor& o, const std::vector<Tensor>& p) {
      const float* saved = act == TALOS_ACT_SILU ? saved_z->dev : o.d();
      check(talos_linear_bwd(ctx(), p[0].d(), p[1].d(), saved, o.g(), p[0].g(), p[1].g(), p.size() > 2 ? p[2].g() : nullptr,
                             (int64_t)rows, (int64_t)in_f, (int64_t)out_f, act, mode(), 7));
    });
    check(talos_linear_fwd(ctx(), x.d(), weight.d(), bias ? bias->d() : nullptr, out.d(), saved_z ? saved_z->dev : nullptr,
                           (int64_t)rows, (int64_t)in_f, (int64_t)out_f, act, mode()));
    return out;
  }
  Tensor forward(const Tensor& x) const override { return forward_act(x, TALOS_ACT_NONE); }
  std::vector<Tensor> parameters() const override { std::vector<Tensor> p{weight}; if (bias) p.push_back(*bias); return p; }
  // Linear::forward_inference (src/nn.rs:37-69): graph-free, slice in / vector out.
  std::vector<double> forward_inference(const std::vector<double>& input) const {
    Tensor x = Tensor::new_(input, {input.size() / in_features, in_features});
    Tensor y = Tensor::zeros({x.shape[0], out_features});
    check(talos_linear_fwd(ctx(), x.d(), weight.d(), bias ? bias->d() : nullptr, y.d(), nullptr, (int64_t)x.shape[0], (int64_t)in_features,
                           (int64_t)out_features, TALOS_ACT_NONE, mode()));
    return y.to_vec();
  }
};

struct RMSNorm : Module {                                                           // src/nn.rs:145-304
  Tensor weight; double eps; size_t dim;
  explicit RMSNorm(Uninit) : eps(0.0), dim(0) {}
  RMSNorm(size_t d, double e, uint64_t /*seed*/) : eps(e), dim(d) { weight = Tensor::new_(std::vector<double>(d, 1.0), {d}); }
  Tensor forward(const Tensor& x) const override {
    TALOS_ASSERT(!x.shape.empty() && x.shape.back() == dim, "RMSNorm dim mismatch");
    const size_t rows = x.len() / dim, dm = dim;
    Buf inv = make_buf(rows, false);
    Tensor out = Tensor::result(x.shape, {x, weight}, [rows, dm, inv](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_rmsnorm_bwd(ctx(), o.g(), p[0].d(), p[1].d(), inv->dev, (int64_t)rows, (int64_t)dm, p[0].g(), p[1].g(), 3));
    });
    check(talos_rmsnorm_fwd(ctx(), x.d(), weight.d(), (float)eps, (int64_t)rows, (int64_t)dim, out.d(), inv->dev));
    return out;
  }
  std::vector<Tensor> parameters() const override { return {weight}; }
  std::vector<double> forward_inference(const std::vector<double>& input) const {   // :160-179
    Tensor x = Tensor::new_(input, {input.size() / dim, dim}); Tensor y = Tensor::zeros(x.shape);
    check(talos_rmsnorm_fwd(ctx(), x.d(), weight.d(), (float)eps, (int64_t)x.shape[0], (int64_t)dim, y.d(), nullptr));
    return y.to_vec();
  }
};

struct RoPE {                                                                       // src/transformer.rs:220-371
  size_t dim; double base = 10000.0; size_t max_len; Buf cos_cache, sin_cache;
  explicit RoPE(Uninit) : dim(0), max_len(0) {}
  RoPE(size_t d, size_t max_l) : dim(d), max_len(max_l) {
    cos_cache = make_buf(max_l * d / 2, false); sin_cache = make_buf(max_l * d / 2, false);
    check(talos_rope_table(ctx(), (int64_t)d, (int64_t)max_l, base, cos_cache->dev, sin_cache->dev));
  }
  // Rotates by the index along shape[len-2] (:262): for [B,S,H,dr] that is the head index.
  Tensor forward(const Tensor& x, size_t start_pos) const {
    TALOS_ASSERT(x.shape.size() >= 2 && x.shape.back() == dim, "RoPE dim mismatch");
    const size_t npos = x.shape[x.shape.size() - 2], outer = x.len() / (npos * dim), dm = dim, tl = max_len * dim / 2;
    TALOS_ASSERT(start_pos + npos <= max_len, "RoPE position beyond the precomputed table");   // the crate indexes out of bounds here
    Buf c = cos_cache, s = sin_cache;
    Tensor out = Tensor::result(x.shape, {x}, [=](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_rope(ctx(), o.g(), p[0].g(), c->dev, s->dev, (int64_t)tl, (int64_t)outer, (int64_t)npos, 1, (int64_t)dm, (int64_t)start_pos, 1, 1));
    });
    check(talos_rope(ctx(), x.d(), out.d(), c->dev, s->dev, (int64_t)tl, (int64_t)outer, (int64_t)npos, 1, (int64_t)dm, (int64_t)start_pos, 0, 0));
    return out;
  }
};

// Token-position rotation of a [B,S,H,dim] tensor (what the graph-free paths do, src/transformer.rs:583-610),
// as a tape node; the crate's own autograd path never rotates this way (see RoPE::forward above).
inline Tensor rope_token(const RoPE& r, const Tensor& x, size_t start_pos) {
  TALOS_ASSERT(x.shape.size() == 4 && x.shape[3] == r.dim, "rope_token expects [B,S,H,dim]");
  const size_t B = x.shape[0], S = x.shape[1], H = x.shape[2], dm = r.dim, tl = r.max_len * r.dim / 2;
  Buf c = r.cos_cache, s = r.sin_cache;
  Tensor out = Tensor::result(x.shape, {x}, [=](const Tensor& o, const std::vector<Tensor>& p) {
    check(talos_rope(ctx(), o.g(), p[0].g(), c->dev, s->dev, (int64_t)tl, (int64_t)B, (int64_t)S, (int64_t)H, (int64_t)dm, (int64_t)start_pos, 1, 1));
  });
  check(talos_rope(ctx(), x.d(), out.d(), c->dev, s->dev, (int64_t)tl, (int64_t)B, (int64_t)S, (int64_t)H, (int64_t)dm, (int64_t)start_pos, 0, 0));
  return out;
}

struct MLAConfig { size_t dim, num_heads, q_lora_rank, kv_lora_rank, qk_rope_dim, v_head_dim, max_seq_len; };   // :9-17

struct KVCache {                                                                    // :400-425, device resident [heads][cap][width]
  size_t num_heads, len = 0, cap = 0, k_width = 0, v_width = 0; Buf k, v;
  explicit KVCache(size_t heads) : num_heads(heads) {}
  void clear() { len = 0; }
};

struct MultiHeadLatentAttention {                                                   // :375-1184
  MLAConfig config; Linear w_dkv, w_uk, w_uv, w_q, w_kr, w_qr, w_o; RoPE rope;
  bool token_positions = false;      // false: the crate's autograd-path behaviour (rotation by head index)
  explicit MultiHeadLatentAttention(Uninit u) : config{}, w_dkv(u), w_uk(u), w_uv(u), w_q(u), w_kr(u), w_qr(u), w_o(u), rope(u) {}
  MultiHeadLatentAttention(const MLAConfig& c, uint64_t seed)
      : config(c), w_dkv(c.dim, c.kv_lora_rank, false, seed), w_uk(c.kv_lora_rank, c.num_heads * c.v_head_dim, false, seed + 1),
        w_uv(c.kv_lora_rank, c.num_heads * c.v_head_dim, false, seed + 2), w_q(c.dim, c.num_heads * c.v_head_dim, false, seed + 3),
        w_kr(c.dim, c.num_heads * c.qk_rope_dim, false, seed + 4), w_qr(c.dim, c.num_heads * c.qk_rope_dim, false, seed + 5),
        w_o(c.num_heads * c.v_head_dim, c.dim, false, seed + 6), rope(c.qk_rope_dim, c.max_seq_len) {}
  std::vector<Tensor> parameters() const {
    std::vector<Tensor> p; for (const Linear* l : {&w_dkv, &w_uk, &w_uv, &w_q, &w_kr, &w_qr, &w_o}) for (auto& t : l->parameters()) p.push_back(t); return p;
  }
  // Fused node for :508-557: concat(content, rope) -> transpose(1,2) -> Q.K^T -> scale -> softmax -> .V -> transpose back.
  static Tensor attention(const Tensor& qc, const Tensor& qr, const Tensor& kc, const Tensor& kr, const Tensor& v, size_t B, size_t S, size_t H,
                          size_t dh, size_t dr, bool causal = false) {
    const size_t tot = dh + dr, BH = B * H; const float scale = 1.f / std::sqrt((float)tot);
    Buf q = make_buf(BH * S * tot, false), k = make_buf(BH * S * tot, false), vv = make_buf(BH * S * dh, false), probs = make_buf(BH * S * S, false);
    auto pack = [&](const Tensor& a, const Tensor* b, size_t wa, size_t wb, float* dst) {   // [B,S,H,wa](+[B,S,H,wb]) -> [B,H,S,wa+wb]
      Buf cat = make_buf(B * S * H * (wa + wb), false);
      if (b && wb) check(talos_concat_last(ctx(), a.d(), b->d(), cat->dev, (int64_t)(B * S * H), (int64_t)wa, (int64_t)wb));
      else check(talos_copy_device(ctx(), cat->dev, a.d(), sizeof(float) * a.len()));
      int64_t shp[4] = {(int64_t)B, (int64_t)S, (int64_t)H, (int64_t)(wa + wb)};
      check(talos_transpose(ctx(), cat->dev, dst, shp, 4, 1, 2, 0));
    };                                                                              // `cat` goes back to the ctx allocator, which hands it only to LATER work on the stream
    pack(qc, &qr, dh, dr, q->dev); pack(kc, &kr, dh, dr, k->dev); pack(v, nullptr, dh, 0, vv->dev);
    Tensor out = Tensor::result({B, S, H * dh}, {qc, qr, kc, kr, v}, [=](const Tensor& o, const std::vector<Tensor>& p) {
      Buf go = make_buf(BH * S * dh, false), gq = make_buf(BH * S * tot, false), gk = make_buf(BH * S * tot, false), gv = make_buf(BH * S * dh, false);
      int64_t bshd[4] = {(int64_t)B, (int64_t)S, (int64_t)H, (int64_t)dh};
      check(talos_transpose(ctx(), o.g(), go->dev, bshd, 4, 1, 2, 0));                // [B,S,H,dh] -> [B,H,S,dh]
      check(talos_attention_bwd(ctx(), q->dev, k->dev, vv->dev, probs->dev, go->dev, gq->dev, gk->dev, gv->dev, (int64_t)BH, (int64_t)S, (int64_t)tot, (int64_t)dh, scale, mode()));
      auto unpack = [&](const float* src, size_t w, float* ga, float* gb, size_t wa, size_t wb) {   // [B,H,S,w] -> [B,S,H,w] -> split, accumulate
        Buf t = make_buf(B * S * H * w, false);
        int64_t bhsw[4] = {(int64_t)B, (int64_t)H, (int64_t)S, (int64_t)w};
        check(talos_transpose(ctx(), src, t->dev, bhsw, 4, 1, 2, 0));
        check(talos_split_last(ctx(), t->dev, ga, gb, (int64_t)(B * S * H), (int64_t)wa, (int64_t)wb, 1));
      };
      unpack(gq->dev, tot, p[0].g(), p[1].g(), dh, dr); unpack(gk->dev, tot, p[2].g(), p[3].g(), dh, dr); unpack(gv->dev, dh, p[4].g(), nullptr, dh, 0);
    });
    Buf att = make_buf(BH * S * dh, false);
    check(talos_attention_fwd(ctx(), q->dev, k->dev, vv->dev, att->dev, probs->dev, (int64_t)BH, (int64_t)S, (int64_t)tot, (int64_t)dh, scale, causal ? 1 : 0, mode()));
    int64_t bhsd[4] = {(int64_t)B, (int64_t)H, (int64_t)S, (int64_t)dh};
    check(talos_transpose(ctx(), att->dev, out.d(), bhsd, 4, 1, 2, 0));
    return out;
  }
  Tensor forward(const Tensor& x) const {                                           // :478-560
    TALOS_ASSERT(x.shape.size() == 3 && x.shape[2] == config.dim, "MLA expects [Batch, Seq, Dim]");
    const size_t B = x.shape[0], S = x.shape[1], H = config.num_heads, dh = config.v_head_dim, dr = config.qk_rope_dim;
    Tensor c_kv = w_dkv.forward(x), k_c = w_uk.forward(c_kv), v_c = w_uv.forward(c_kv);
    Tensor k_r = w_kr.forward(x).reshape({B, S, H, dr}), q_c = w_q.forward(x), q_r = w_qr.forward(x).reshape({B, S, H, dr});
    Tensor k_rot = token_positions ? rope_token(rope, k_r, 0) : rope.forward(k_r, 0);   // head-index positions are what the crate does here
    Tensor q_rot = token_positions ? rope_token(rope, q_r, 0) : rope.forward(q_r, 0);
    Tensor att = attention(q_c, q_rot, k_c, k_rot, v_c, B, S, H, dh, dr);
    return w_o.forward(att);
  }
  // forward_inference (:562-685): graph-free forward of ONE whole sequence [seq, dim], token-position RoPE, every token
  // attending to every token -- which is what the cached variant below computes when it is handed the whole sequence
  // and an empty cache.
  std::vector<double> forward_inference(const std::vector<double>& xin) const { KVCache fresh(config.num_heads); return forward_inference_cached(xin, fresh, 0); }
  // forward_inference_cached (:688-841): `x` holds one or a few tokens of ONE sequence; token-position RoPE;
  // K/V rows are appended to the cache and the new tokens attend to every cached row.
  std::vector<double> forward_inference_cached(const std::vector<double>& xin, KVCache& cache, size_t start_pos) const {
    const size_t D = config.dim, H = config.num_heads, dh = config.v_head_dim, dr = config.qk_rope_dim, tot = dh + dr, S = xin.size() / D;
    Tensor x = Tensor::new_(xin, {S, D});
    auto lin = [&](const Linear& l, const Tensor& in) { Tensor y = Tensor::zeros({S, l.out_features});
      check(talos_linear_fwd(ctx(), in.d(), l.weight.d(), nullptr, y.d(), nullptr, (int64_t)S, (int64_t)l.in_features, (int64_t)l.out_features, 0, mode())); return y; };
    Tensor c_kv = lin(w_dkv, x), k_c = lin(w_uk, c_kv), v_c = lin(w_uv, c_kv), k_r = lin(w_kr, x), q_c = lin(w_q, x), q_r = lin(w_qr, x);
    const size_t tl = rope.max_len * dr / 2;
    check(talos_rope(ctx(), k_r.d(), k_r.d(), rope.cos_cache->dev, rope.sin_cache->dev, (int64_t)tl, 1, (int64_t)S, (int64_t)H, (int64_t)dr, (int64_t)start_pos, 0, 0));
    check(talos_rope(ctx(), q_r.d(), q_r.d(), rope.cos_cache->dev, rope.sin_cache->dev, (int64_t)tl, 1, (int64_t)S, (int64_t)H, (int64_t)dr, (int64_t)start_pos, 0, 0));
    Tensor q = Tensor::zeros({S, H, tot}), k = Tensor::zeros({S, H, tot});
    check(talos_concat_last(ctx(), q_c.d(), q_r.d(), q.d(), (int64_t)(S * H), (int64_t)dh, (int64_t)dr));
    check(talos_concat_last(ctx(), k_c.d(), k_r.d(), k.d(), (int64_t)(S * H), (int64_t)dh, (int64_t)dr));
    // grow the cache ([H][cap][w]) and append the new rows head by head
    if (cache.len + S > cache.cap) {
      size_t ncap = std::max<size_t>(16, 2 * (cache.len + S)); Buf nk = make_buf(H * ncap * tot), nv = make_buf(H * ncap * dh);
      for (size_t h = 0; h < H && cache.len; ++h) {
        check(talos_copy_device(ctx(), nk->dev + h * ncap * tot, cache.k->dev + h * cache.cap * tot, sizeof(float) * cache.len * tot));
        check(talos_copy_device(ctx(), nv->dev + h * ncap * dh, cache.v->dev + h * cache.cap * dh, sizeof(float) * cache.len * dh));
      }
      cache.k = nk; cache.v = nv; cache.cap = ncap; cache.k_width = tot; cache.v_width = dh;
    }
    for (size_t t = 0; t < S; ++t) for (size_t h = 0; h < H; ++h) {
      check(talos_copy_device(ctx(), cache.k->dev + (h * cache.cap + cache.len + t) * tot, k.d() + (t * H + h) * tot, sizeof(float) * tot));
      check(talos_copy_device(ctx(), cache.v->dev + (h * cache.cap + cache.len + t) * dh, v_c.d() + (t * H + h) * dh, sizeof(float) * dh));
    }
    cache.len += S;
    const size_t L = cache.len;
    Tensor scores = Tensor::zeros({H, S, L}), att = Tensor::zeros({S, H * dh});
    // scores[h] = q[:,h,:] . Kcache[h]^T ; softmax(scale * scores) ; att[:,h,:] = P[h] . Vcache[h]
    check(talos_gemm_batched(ctx(), TALOS_OP_N, TALOS_OP_T, (int64_t)S, (int64_t)L, (int64_t)tot, q.d(), (int64_t)(H * tot), (int64_t)tot, cache.k->dev, (int64_t)tot,
                             (int64_t)(cache.cap * tot), scores.d(), (int64_t)L, (int64_t)(S * L), (int64_t)H, 0, TALOS_MODE_FP32));
    check(talos_softmax_fwd(ctx(), scores.d(), scores.d(), (int64_t)(H * S), (int64_t)L, 1.f / std::sqrt((float)tot), 0));
    check(talos_gemm_batched(ctx(), TALOS_OP_N, TALOS_OP_N, (int64_t)S, (int64_t)dh, (int64_t)L, scores.d(), (int64_t)L, (int64_t)(S * L), cache.v->dev, (int64_t)dh,
                             (int64_t)(cache.cap * dh), att.d(), (int64_t)(H * dh), (int64_t)dh, (int64_t)H, 0, TALOS_MODE_FP32));
    Tensor y = lin(w_o, att);
    return y.to_vec();
  }
  void prune_kv_cache(KVCache& cache, size_t max_seq_len) const {                   // :843-874
    if (!cache.k || cache.len <= max_seq_len) return;
    const size_t rm = cache.len - max_seq_len, tot = cache.k_width, dh = cache.v_width;
    Buf nk = make_buf(cache.num_heads * cache.cap * tot), nv = make_buf(cache.num_heads * cache.cap * dh);
    for (size_t h = 0; h < cache.num_heads; ++h) {
      check(talos_copy_device(ctx(), nk->dev + h * cache.cap * tot, cache.k->dev + (h * cache.cap + rm) * tot, sizeof(float) * max_seq_len * tot));
      check(talos_copy_device(ctx(), nv->dev + h * cache.cap * dh, cache.v->dev + (h * cache.cap + rm) * dh, sizeof(float) * max_seq_len * dh));
    }
    cache.k = nk; cache.v = nv; cache.len = max_seq_len;
  }
};

struct LuckTransformer : Module {                                                   // src/transformer.rs:36-216
  Linear embed; RMSNorm norm_1; MultiHeadLatentAttention mla_layer; RMSNorm norm_2; Linear ffn_1, ffn_2; RMSNorm norm_final; Linear out_proj;
  explicit LuckTransformer(Uninit u) : embed(u), norm_1(u), mla_layer(u), norm_2(u), ffn_1(u), ffn_2(u), norm_final(u), out_proj(u) {}
  LuckTransformer(size_t in_dim, size_t hidden, bool /*bias*/, uint64_t seed)
      : embed(in_dim, hidden, true, seed), norm_1(hidden, 1e-5, seed + 5), mla_layer(MLAConfig{hidden, 4, 0, 32, 16, hidden / 4, 256}, seed + 10),
        norm_2(hidden, 1e-5, seed + 15), ffn_1(hidden, hidden * 2, true, seed + 20), ffn_2(hidden * 2, hidden, true, seed + 30),
        norm_final(hidden, 1e-5, seed + 35), out_proj(hidden, hidden, true, seed + 40) {}
  Tensor forward(const Tensor& x) const override {                                  // :71-90
    Tensor h = embed.forward(x);
    Tensor h2 = h + mla_layer.forward(norm_1.forward(h));
    Tensor f1 = ffn_1.forward_act(norm_2.forward(h2), TALOS_ACT_RELU);              // relu fused into the Linear node
    Tensor h3 = h2 + ffn_2.forward(f1);
    return out_proj.forward(norm_final.forward(h3));
  }
  // last_token (:92-109): returns a NEW LEAF -- it cuts the graph, as the crate does.
  Tensor last_token(const Tensor& x) const {
    TALOS_ASSERT(x.shape.size() == 3, "last_token expects [Batch, Seq, Dim]");
    Tensor out = Tensor::zeros({x.shape[0], x.shape[2]});
    check(talos_last_token(ctx(), x.d(), out.d(), (int64_t)x.shape[0], (int64_t)x.shape[1], (int64_t)x.shape[2]));
    return out;
  }
  std::vector<double> forward_inference(const std::vector<double>& x) const {       // :111-144: one whole sequence, graph-free
    KVCache fresh(mla_layer.config.num_heads); return forward_inference_step(x, fresh, 0);
  }
  std::vector<double> last_token_inference(const std::vector<double>& x) const {    // :146-150
    const size_t dim = out_proj.out_features, start = x.size() > dim ? x.size() - dim : 0;
    return std::vector<double>(x.begin() + start, x.end());
  }
  std::vector<double> forward_inference_step(const std::vector<double>& x, KVCache& cache, size_t start_pos) const {   // :152-193
    auto add = [](std::vector<double> a, const std::vector<double>& b) { for (size_t i = 0; i < a.size(); ++i) a[i] += b[i]; return a; };
    std::vector<double> h = embed.forward_inference(x);
    std::vector<double> h2 = add(h, mla_layer.forward_inference_cached(norm_1.forward_inference(h), cache, start_pos));
    std::vector<double> f1 = ffn_1.forward_inference(norm_2.forward_inference(h2));
    for (double& v : f1) if (v < 0.0) v = 0.0;
    std::vector<double> h3 = add(h2, ffn_2.forward_inference(f1));
    return out_proj.forward_inference(norm_final.forward_inference(h3));
  }
  std::vector<Tensor> parameters() const override {
    std::vector<Tensor> p; auto ext = [&](std::vector<Tensor> v) { p.insert(p.end(), v.begin(), v.end()); };
    ext(embed.parameters()); ext(norm_1.parameters()); ext(mla_layer.parameters()); ext(norm_2.parameters()); ext(ffn_1.parameters());
    ext(ffn_2.parameters()); ext(norm_final.parameters()); ext(out_proj.parameters()); return p;
  }
};

// Slices [rows, wa+wb] into ([rows, wa], [rows, wb]) as a tape node (backward = concat of the two gradients).
inline std::pair<Tensor, Tensor> split_last(const Tensor& x, size_t wa, size_t wb) {
  TALOS_ASSERT(!x.shape.empty() && x.shape.back() == wa + wb, "split_last width mismatch");
  const size_t rows = x.len() / (wa + wb);
  std::vector<size_t> sa = x.shape, sb = x.shape; sa.back() = wa; sb.back() = wb;
  // one shared node would need two outputs; two nodes, each scattering its own gradient slice, give the same sums
  Tensor a = Tensor::result(sa, {x}, [rows, wa, wb](const Tensor& o, const std::vector<Tensor>& p) {
    Buf z = make_buf(rows * wb); Buf cat = make_buf(rows * (wa + wb), false);
    check(talos_concat_last(ctx(), o.g(), z->dev, cat->dev, (int64_t)rows, (int64_t)wa, (int64_t)wb));
    check(talos_eltwise_binary(ctx(), TALOS_EW_ADD, p[0].g(), cat->dev, p[0].g(), (int64_t)(rows * (wa + wb))));
  });
  Tensor b = Tensor::result(sb, {x}, [rows, wa, wb](const Tensor& o, const std::vector<Tensor>& p) {
    Buf z = make_buf(rows * wa); Buf cat = make_buf(rows * (wa + wb), false);
    check(talos_concat_last(ctx(), z->dev, o.g(), cat->dev, (int64_t)rows, (int64_t)wa, (int64_t)wb));
    check(talos_eltwise_binary(ctx(), TALOS_EW_ADD, p[0].g(), cat->dev, p[0].g(), (int64_t)(rows * (wa + wb))));
  });
  check(talos_split_last(ctx(), x.d(), a.d(), b.d(), (int64_t)rows, (int64_t)wa, (int64_t)wb, 0));
  return {a, b};
}

// Plain pre-norm multi-head block (not in the crate; the benchmark's config 3) in the crate's residual order
// (src/transformer.rs:71-90): RMSNorm -> QKV -> RoPE(token) -> causal attention -> W_o -> +res -> RMSNorm -> W_ff1 ->
// SiLU -> W_ff2 -> +res.  No biases.
struct TransformerBlock : Module {
  size_t dim, heads; RMSNorm norm_1, norm_2; Linear w_qkv, w_o, w_ff1, w_ff2; RoPE rope;
  TransformerBlock(size_t d, size_t h, size_t ff, size_t max_seq, double eps, uint64_t seed)
      : dim(d), heads(h), norm_1(d, eps, seed), norm_2(d, eps, seed + 1), w_qkv(d, 3 * d, false, seed + 2), w_o(d, d, false, seed + 3),
        w_ff1(d, ff, false, seed + 4), w_ff2(ff, d, false, seed + 5), rope(d / h, max_seq) {}
  Tensor forward(const Tensor& x) const override {
    TALOS_ASSERT(x.shape.size() == 3 && x.shape[2] == dim, "TransformerBlock expects [Batch, Seq, Dim]");
    const size_t B = x.shape[0], S = x.shape[1], dh = dim / heads;
    Tensor qkv = w_qkv.forward(norm_1.forward(x));                                  // [B,S,3*dim] laid out [q | k | v]
    auto [q, kv] = split_last(qkv, dim, 2 * dim);
    auto [k, v] = split_last(kv, dim, dim);
    Tensor qr = rope_token(rope, q.reshape({B, S, heads, dh}), 0), kr = rope_token(rope, k.reshape({B, S, heads, dh}), 0);
    Tensor none = Tensor::zeros({1});
    Tensor att = MultiHeadLatentAttention::attention(qr, none, kr, none, v, B, S, heads, dh, 0, true);
    Tensor h2 = x + w_o.forward(att);
    Tensor f = w_ff1.forward_act(norm_2.forward(h2), TALOS_ACT_SILU);
    return h2 + w_ff2.forward(f);
  }
  std::vector<Tensor> parameters() const override { return {norm_1.weight, w_qkv.weight, w_o.weight, norm_2.weight, w_ff1.weight, w_ff2.weight}; }
};

struct ActorCritic {                                                                // src/ppo.rs:247-307
  static constexpr size_t DIM = 8, ACTION_SPACE = 5;                                // src/neural.rs:3, src/ppo.rs:15
  LuckTransformer backbone; Linear actor_head, critic_head;
  explicit ActorCritic(Uninit u) : backbone(u), actor_head(u), critic_head(u) {}
  explicit ActorCritic(uint64_t seed) : backbone(DIM, 64, true, seed), actor_head(64, ACTION_SPACE, true, seed + 100), critic_head(64, 1, true, seed + 200) {}
  Tensor head(const Tensor& state, const Linear& h) const {
    Tensor x = state.shape.size() == 1 ? state.reshape({1, 1, state.shape[0]}) : state.shape.size() == 2 ? state.reshape({1, state.shape[0], state.shape[1]}) : state;
    Tensor out = h.forward(backbone.last_token(backbone.forward(x)));
    return (out.shape.size() == 2 && out.shape[0] == 1) ? out.reshape({out.shape[1]}) : out;
  }
  Tensor forward_actor(const Tensor& state) const { return head(state, actor_head); }    // :266-282
  Tensor forward_critic(const Tensor& state) const { return head(state, critic_head); }  // :284-300
  std::vector<Tensor> parameters() const { auto p = backbone.parameters(); for (auto& t : actor_head.parameters()) p.push_back(t); for (auto& t : critic_head.parameters()) p.push_back(t); return p; }
};

// DuelingQNetwork (src/dqn.rs:46-160): 8 -> 64 -> 64 -> {value 1, advantage 5}, ReLU, Q = V + A - mean(A).
// The crate spells the combination as three matmuls with constant ones matrices; here it is one fused tape node.
struct DuelingQNetwork : Module {
  static constexpr size_t DIM = 8, ACTION_SPACE = 5;
  Linear l1, l2, val_head, adv_head;
  explicit DuelingQNetwork(uint64_t seed) : l1(DIM, 64, true, seed), l2(64, 64, true, seed + 1), val_head(64, 1, true, seed + 2), adv_head(64, ACTION_SPACE, true, seed + 3) {}   // :55-58
  Tensor forward(const Tensor& state) const override {                              // forward_impl :68-107 (both branches compute the same thing)
    const bool single = state.shape.size() == 1;
    Tensor s2 = single ? state.reshape({1, state.shape[0]}) : state;
    Tensor x = l2.forward_act(l1.forward_act(s2, TALOS_ACT_RELU), TALOS_ACT_RELU);
    Tensor val = val_head.forward(x), adv = adv_head.forward(x);
    const size_t B = adv.shape[0], A = adv.shape[1];
    Tensor q = Tensor::result({B, A}, {val, adv}, [B, A](const Tensor& o, const std::vector<Tensor>& p) {
      check(talos_dueling_combine_bwd(ctx(), o.g(), p[0].g(), p[1].g(), (int64_t)B, (int64_t)A, 1));
    });
    check(talos_dueling_combine_fwd(ctx(), val.d(), adv.d(), q.d(), (int64_t)B, (int64_t)A));
    return single ? q.reshape({A}) : q;
  }
  std::vector<Tensor> parameters() const override {
    std::vector<Tensor> p; for (const Linear* l : {&l1, &l2, &val_head, &adv_head}) for (auto& t : l->parameters()) p.push_back(t); return p;
  }
  void load_state_dict(const DuelingQNetwork& other) {                              // :112-127
    auto a = parameters(), b = other.parameters();
    for (size_t i = 0; i < a.size(); ++i) check(talos_copy_device(ctx(), a[i].d(), b[i].d(), sizeof(float) * a[i].len()));
  }
  void soft_update(const DuelingQNetwork& source, double tau) {                     // :129-150
    auto a = parameters(), b = source.parameters();
    for (size_t i = 0; i < a.size(); ++i) check(talos_soft_update(ctx(), a[i].d(), b[i].d(), (float)tau, (int64_t)a[i].len()));
  }
  size_t predict_action(const Tensor& state) const {                                // :152-170: first maximum
    const std::vector<double> q = forward(state).to_vec();
    size_t best = 0; double mx = -INFINITY;
    for (size_t i = 0; i < q.size(); ++i) if (q[i] > mx) { mx = q[i]; best = i; }
    return best;
  }
};

// The loss of one DQN train step (src/dqn.rs:516-561) as a tape node on the policy network's Q values: double-DQN
// targets from the two networks' next-state Q values, Q of the taken actions, mean squared error.
inline Tensor dqn_loss(const Tensor& q, const std::vector<int32_t>& actions, const Tensor& q_next_eval, const Tensor& q_next_target,
                       const std::vector<double>& rewards, const std::vector<double>& dones, double gamma = 0.99) {
  const size_t B = q.shape[0], A = q.shape[1];
  TALOS_ASSERT(actions.size() == B && rewards.size() == B && dones.size() == B && q_next_eval.len() == B * A && q_next_target.len() == B * A, "DQN batch size mismatch");
  Tensor r = Tensor::new_(rewards, {B}), d = Tensor::new_(dones, {B}), target = Tensor::zeros({B});
  Buf act = make_buf(B, false), dq = make_buf(B * A, false);
  check(talos_copy_from_host(ctx(), act->dev, actions.data(), sizeof(int32_t) * B));
  check(talos_dqn_target(ctx(), q_next_eval.d(), q_next_target.d(), r.d(), d.d(), (float)gamma, target.d(), (int64_t)B, (int64_t)A));
  Tensor loss = Tensor::result({1}, {q}, [dq, B, A](const Tensor& o, const std::vector<Tensor>& p) {
    // dq holds dloss/dq for an upstream gradient of 1; scale by the actual one (1.0 when loss.backward() starts here)
    Buf scaled = make_buf(B * A, false);
    check(talos_fill_from_scalar(ctx(), o.g(), 1.f, scaled->dev, (int64_t)(B * A), 0));
    check(talos_eltwise_binary(ctx(), TALOS_EW_MUL, scaled->dev, dq->dev, scaled->dev, (int64_t)(B * A)));
    check(talos_eltwise_binary(ctx(), TALOS_EW_ADD, p[0].g(), scaled->dev, p[0].g(), (int64_t)(B * A)));
  });
  check(talos_dqn_loss_fwd_bwd(ctx(), q.d(), (const int32_t*)act->dev, target.d(), loss.d(), dq->dev, (int64_t)B, (int64_t)A));
  return loss;                                                                      // `act`, r, d go back to the stream-ordered allocator
}

// RunningMeanStd (src/ppo.rs:444-480): host arithmetic in f64 exactly as the crate (a few scalars per reward).
struct RunningMeanStd {
  double count = 1e-4, mean = 0.0, var = 1.0;
  void update(double x) {
    const double delta = x - mean, tot = count + 1.0;
    const double m2 = var * count + delta * delta * count / tot;
    mean += delta / tot; var = m2 / tot; count = tot;
  }
  double normalize(double x) const { return (x - mean) / (std::sqrt(var) + 1e-8); }
};

// The advantage block of PPO::update (src/ppo.rs:650-675) on the device: normalised, clipped rewards -> reverse GAE
// scan -> returns; advantages normalised with the population standard deviation.  Returns {norm_advantages, returns}.
inline std::pair<Tensor, Tensor> gae_advantages(const Tensor& rewards, const Tensor& values, const std::vector<int32_t>& is_terminals,
                                                const RunningMeanStd& reward_normalizer, double gamma = 0.99, double lambda = 0.95) {
  const size_t len = rewards.len();
  TALOS_ASSERT(values.len() == len && is_terminals.size() == len, "rollout buffers must have one entry per step");
  Tensor adv = Tensor::zeros({len}), ret = Tensor::zeros({len});
  if (len == 0) return {adv, ret};
  Buf term = make_buf(len, false);
  check(talos_copy_from_host(ctx(), term->dev, is_terminals.data(), sizeof(int32_t) * len));
  check(talos_gae(ctx(), rewards.d(), values.d(), (const int32_t*)term->dev, (int64_t)len, (float)gamma, (float)lambda, (float)reward_normalizer.mean,
                  (float)reward_normalizer.var, adv.d(), ret.d()));
  check(talos_normalize_slice(ctx(), adv.d(), (int64_t)len, adv.d(), nullptr));
  return {adv, ret};
}

// ActorCritic::step_inference_cached (src/ppo.rs:391-432) for N simulations at once: what the simulator does once
// per pull and per simulation (src/sim.rs:208, then prune_cache at :578) becomes one GEMM per layer over all
// simulations plus one attention kernel over per-simulation KV rings.  Graph-free; every buffer is allocated once.
// A ring of context_len + 1 slots reproduces "append, attend, prune to context_len".  Sampling stays with the
// caller (the crate uses rand::random there): step() returns the action probabilities.
struct BatchedRollout {
  const ActorCritic& ac; size_t n, context_len, cap;
  Buf k_cache, v_cache, pos, reset_dev;                       // pos / reset_dev hold int32 values
  Buf x, h, hn, c_kv, k_c, v_c, k_r, q_c, q_r, att, ao, h2, f1, f2, h3, o, logits, probs;
  BatchedRollout(const ActorCritic& policy, size_t sims, size_t ctx_len) : ac(policy), n(sims), context_len(ctx_len), cap(ctx_len + 1) {
    const MLAConfig& c = ac.backbone.mla_layer.config;
    const size_t H = c.num_heads, dh = c.v_head_dim, dr = c.qk_rope_dim, D = c.dim;
    k_cache = make_buf(n * H * cap * (dh + dr)); v_cache = make_buf(n * H * cap * dh); pos = make_buf(n); reset_dev = make_buf(n);
    x = make_buf(n * ActorCritic::DIM, false); h = make_buf(n * D, false); hn = make_buf(n * D, false); c_kv = make_buf(n * c.kv_lora_rank, false);
    k_c = make_buf(n * H * dh, false); v_c = make_buf(n * H * dh, false); q_c = make_buf(n * H * dh, false);
    k_r = make_buf(n * H * dr, false); q_r = make_buf(n * H * dr, false); att = make_buf(n * H * dh, false); ao = make_buf(n * D, false);
    h2 = make_buf(n * D, false); f1 = make_buf(n * 2 * D, false); f2 = make_buf(n * D, false); h3 = make_buf(n * D, false); o = make_buf(n * D, false);
    logits = make_buf(n * ActorCritic::ACTION_SPACE, false); probs = make_buf(n * ActorCritic::ACTION_SPACE, false);
  }
  void reset_all() { check(talos_memset_zero(ctx(), pos->dev, sizeof(float) * n)); }     // every simulation starts a new episode
  // One policy step for all simulations.  `states_dev`: [N, DIM] fp32 on the device.  `reset_after` (nullable, N
  // entries): simulations whose episode ends with this step.  Returns the device buffer of probabilities [N, A].
  const float* step(const float* states_dev, const std::vector<int32_t>* reset_after = nullptr) {
    const LuckTransformer& t = ac.backbone; const MultiHeadLatentAttention& m = t.mla_layer; const MLAConfig& c = m.config;
    const size_t H = c.num_heads, dh = c.v_head_dim, dr = c.qk_rope_dim, D = c.dim;
    auto lin = [&](const Linear& l, const float* in, float* out, int act = TALOS_ACT_NONE) {
      check(talos_linear_fwd(ctx(), in, l.weight.d(), l.bias ? l.bias->d() : nullptr, out, nullptr, (int64_t)n, (int64_t)l.in_features, (int64_t)l.out_features, act, mode()));
    };
    auto norm = [&](const RMSNorm& r, const float* in, float* out) {
      check(talos_rmsnorm_fwd(ctx(), in, r.weight.d(), (float)r.eps, (int64_t)n, (int64_t)r.dim, out, nullptr));
    };
    lin(t.embed, states_dev, h->dev);                                                 // src/transformer.rs:159-160
    norm(t.norm_1, h->dev, hn->dev);
    lin(m.w_dkv, hn->dev, c_kv->dev); lin(m.w_uk, c_kv->dev, k_c->dev); lin(m.w_uv, c_kv->dev, v_c->dev);   // :705-710
    lin(m.w_kr, hn->dev, k_r->dev); lin(m.w_q, hn->dev, q_c->dev); lin(m.w_qr, hn->dev, q_r->dev);
    check(talos_mla_decode_step(ctx(), q_c->dev, q_r->dev, k_c->dev, k_r->dev, v_c->dev, m.rope.cos_cache->dev, m.rope.sin_cache->dev,
                                (int64_t)(m.rope.max_len * dr / 2), (const int32_t*)pos->dev, k_cache->dev, v_cache->dev, att->dev, (int64_t)n, (int64_t)H,
                                (int64_t)dh, (int64_t)dr, (int64_t)cap, 1.f / std::sqrt((float)(dh + dr))));
    lin(m.w_o, att->dev, ao->dev);
    check(talos_eltwise_binary(ctx(), TALOS_EW_ADD, h->dev, ao->dev, h2->dev, (int64_t)(n * D)));            // :166-170
    norm(t.norm_2, h2->dev, hn->dev);
    lin(t.ffn_1, hn->dev, f1->dev, TALOS_ACT_RELU); lin(t.ffn_2, f1->dev, f2->dev);                          // :174-183
    check(talos_eltwise_binary(ctx(), TALOS_EW_ADD, h2->dev, f2->dev, h3->dev, (int64_t)(n * D)));
    norm(t.norm_final, h3->dev, hn->dev);
    lin(t.out_proj, hn->dev, o->dev);
    lin(ac.actor_head, o->dev, logits->dev);                                          // src/ppo.rs:400
    check(talos_softmax_fwd(ctx(), logits->dev, probs->dev, (int64_t)n, (int64_t)ActorCritic::ACTION_SPACE, 1.f, 0));
    const int32_t* rs = nullptr;
    if (reset_after) {
      TALOS_ASSERT(reset_after->size() == n, "reset mask must have one entry per simulation");
      check(talos_copy_from_host(ctx(), reset_dev->dev, reset_after->data(), sizeof(int32_t) * n));
      rs = (const int32_t*)reset_dev->dev;
    }
    check(talos_decode_advance(ctx(), (int32_t*)pos->dev, rs, (int64_t)n));
    return probs->dev;
  }
  std::vector<double> step_host(const std::vector<double>& states, const std::vector<int32_t>* reset_after = nullptr) {
    TALOS_ASSERT(states.size() == n * ActorCritic::DIM, "states must be [N, DIM]");
    check(talos_upload_f64(ctx(), x->dev, states.data(), (int64_t)states.size()));
    const float* p = step(x->dev, reset_after);
    std::vector<double> out(n * ActorCritic::ACTION_SPACE);
    check(talos_download_f64(ctx(), out.data(), p, (int64_t)out.size()));
    return out;
  }
};

struct Adam {                                                                       // src/ppo.rs:482-540; clip_norm = 1 gives src/dqn.rs:207-239
  std::vector<Tensor> params; std::vector<Buf> m, v; Buf sumsq; size_t t = 0; double lr, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, clip_norm = 0.0;
  Adam(std::vector<Tensor> p, double learning_rate) : params(std::move(p)), lr(learning_rate) { for (auto& q : params) { m.push_back(make_buf(q.len())); v.push_back(make_buf(q.len())); } }
  void set_lr(double l) { lr = l; }
  void step() {
    ++t;
    if (clip_norm > 0.0) {                                                          // global norm over ALL parameters first, on the device
      if (!sumsq) sumsq = make_buf(1);
      check(talos_memset_zero(ctx(), sumsq->dev, sizeof(float)));
      for (auto& p : params) check(talos_dot(ctx(), p.g(), p.g(), (int64_t)p.len(), sumsq->dev, 1));
      for (size_t i = 0; i < params.size(); ++i)
        check(talos_adam_step_global_clip(ctx(), params[i].d(), params[i].g(), m[i]->dev, v[i]->dev, (int64_t)params[i].len(), (int64_t)t, (float)lr, (float)beta1,
                                          (float)beta2, (float)eps, 1.f, sumsq->dev, (float)clip_norm));
      return;
    }
    for (size_t i = 0; i < params.size(); ++i)
      check(talos_adam_step(ctx(), params[i].d(), params[i].g(), m[i]->dev, v[i]->dev, (int64_t)params[i].len(), (int64_t)t, (float)lr, (float)beta1, (float)beta2,
                            (float)eps, 1.f, 0.f));
  }
  void zero_grad() const { for (auto& p : params) p.zero_grad(); }
};

}  // namespace talos
