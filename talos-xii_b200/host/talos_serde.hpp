// The model files of the reference crate, so that a policy cached by one implementation loads in the other.
//
// save_ppo_model / load_ppo_model (src/main.rs:123-166) write `<path>.bin` with bincode 1.x (default options) and
// `<path>` with serde_json (compact), both driven by the serde derives of the model structs; load tries the binary
// file first and falls back to JSON.  What those derives produce, field by field, in declaration order:
//
//   ActorCritic { backbone: LuckTransformer, actor_head: Linear, critic_head: Linear }          src/ppo.rs:246-252
//   LuckTransformer { embed: Linear, norm_1: RMSNorm, mla_layer: MultiHeadLatentAttention, norm_2: RMSNorm,
//                     ffn_1: Linear, ffn_2: Linear, norm_final: RMSNorm, out_proj: Linear }       src/transformer.rs:35-46
//   MultiHeadLatentAttention { config: MLAConfig, w_dkv, w_uk, w_uv, w_q, w_kr, w_qr, w_o: Linear, rope: RoPE }   :374-398
//   MLAConfig { dim, num_heads, q_lora_rank, kv_lora_rank, qk_rope_dim, v_head_dim, max_seq_len: usize }          :8-17
//   RoPE { dim: usize, base: f64, cos_cache: Vec<f64>, sin_cache: Vec<f64> }                      :219-225
//   Linear { weight: Tensor, bias: Option<Tensor>, in_features: usize, out_features: usize }      src/nn.rs:11-17
//   RMSNorm { weight: Tensor, eps: f64, dim: usize }                                              src/nn.rs:144-149
//   Tensor { data: Vec<f64>, shape: Vec<usize> }   (hand-written impl)                            src/autograd.rs:22-50
//
// bincode 1.x defaults: little-endian, fixed-width integers; usize as u64; f64 as 8 bytes; Vec<T> as u64 length + the
// elements; Option<T> as one byte 0 / 1 followed by T; a struct is its fields back to back, no names, no framing.
// serde_json: a struct is an object with the field names as keys in declaration order, None is null, usize is a plain
// integer, f64 is the shortest decimal that round-trips, written the way the `ryu` crate prints it (always with a
// fraction or an exponent: 1.0, 10000.0, 0.00001, 1e-6, 1.2345e-7), non-finite values are null.
//
// No file written by the reference exists here to compare with (the crate cannot be built in this image); the byte
// layouts are checked against files assembled by hand from the rules above.
#pragma once
#include <charconv>
#include <fstream>

#include "talos.hpp"

namespace talos {
namespace serde {

// ------------------------------------------------------------------ bincode
struct BinWriter {
  std::vector<uint8_t> buf;
  void u8(uint8_t x) { buf.push_back(x); }
  void u64(uint64_t x) { uint8_t b[8]; std::memcpy(b, &x, 8); buf.insert(buf.end(), b, b + 8); }
  void f64(double x) { uint8_t b[8]; std::memcpy(b, &x, 8); buf.insert(buf.end(), b, b + 8); }
  void vec_f64(const std::vector<double>& v) { u64(v.size()); const uint8_t* p = (const uint8_t*)v.data(); buf.insert(buf.end(), p, p + 8 * v.size()); }
};
struct BinReader {
  const std::vector<uint8_t>& buf; size_t o = 0;
  explicit BinReader(const std::vector<uint8_t>& b) : buf(b) {}
  void need(size_t n) const { TALOS_ASSERT(o + n <= buf.size() && o + n >= o, "model file is truncated"); }
  uint8_t u8() { need(1); return buf[o++]; }
  uint64_t u64() { need(8); uint64_t x; std::memcpy(&x, buf.data() + o, 8); o += 8; return x; }
  double f64() { need(8); double x; std::memcpy(&x, buf.data() + o, 8); o += 8; return x; }
  std::vector<double> vec_f64() {
    const uint64_t n = u64(); TALOS_ASSERT(n <= (buf.size() - o) / 8, "model file is truncated");
    std::vector<double> v(n); std::memcpy(v.data(), buf.data() + o, 8 * n); o += 8 * n; return v;
  }
  std::vector<size_t> vec_usize() {
    const uint64_t n = u64(); TALOS_ASSERT(n <= 8, "tensor rank out of range");
    std::vector<size_t> v(n); for (auto& d : v) d = (size_t)u64(); return v;
  }
};

// RoPE's tables as the crate computes and stores them: f64, position-major (src/transformer.rs:239-251).
inline void rope_tables_f64(size_t dim, size_t max_len, double base, std::vector<double>* c, std::vector<double>* s) {
  c->clear(); s->clear(); c->reserve(max_len * (dim / 2)); s->reserve(max_len * (dim / 2));
  for (size_t pos = 0; pos < max_len; ++pos)
    for (size_t i = 0; i < dim / 2; ++i) {
      const double theta = 1.0 / std::pow(base, (double)(2 * i) / (double)dim), angle = (double)pos * theta;
      c->push_back(std::cos(angle)); s->push_back(std::sin(angle));
    }
}
// The tables of a loaded RoPE go to the device as they are in the file (rounded to fp32).
inline void rope_from_tables(RoPE* r, size_t dim, double base, const std::vector<double>& c, const std::vector<double>& s) {
  TALOS_ASSERT(dim >= 2 && dim % 2 == 0 && c.size() == s.size() && c.size() % (dim / 2) == 0, "RoPE tables do not match the rotary dimension");
  r->dim = dim; r->base = base; r->max_len = c.size() / (dim / 2);
  r->cos_cache = make_buf(c.size(), false); r->sin_cache = make_buf(s.size(), false);
  check(talos_upload_f64(ctx(), r->cos_cache->dev, c.data(), (int64_t)c.size()));
  check(talos_upload_f64(ctx(), r->sin_cache->dev, s.data(), (int64_t)s.size()));
}

inline void write(BinWriter& w, const Tensor& t) { w.vec_f64(t.to_vec()); w.u64(t.shape.size()); for (size_t d : t.shape) w.u64(d); }
inline Tensor read_tensor(BinReader& r) {
  std::vector<double> v = r.vec_f64(); std::vector<size_t> shp = r.vec_usize();
  TALOS_ASSERT(numel(shp) == v.size(), "Data length must match shape");           // Tensor::new's assertion (src/autograd.rs:96-100)
  return Tensor::new_(v, std::move(shp));
}
inline void write(BinWriter& w, const Linear& l) {
  write(w, l.weight);
  if (l.bias) { w.u8(1); write(w, *l.bias); } else w.u8(0);
  w.u64(l.in_features); w.u64(l.out_features);
}
inline void read(BinReader& r, Linear* l) {
  l->weight = read_tensor(r);
  const uint8_t tag = r.u8(); TALOS_ASSERT(tag <= 1, "bad Option tag in model file");
  if (tag) l->bias = read_tensor(r); else l->bias.reset();
  l->in_features = (size_t)r.u64(); l->out_features = (size_t)r.u64();
  TALOS_ASSERT(l->weight.shape == (std::vector<size_t>{l->in_features, l->out_features}), "Linear weight shape does not match its feature counts");
}
inline void write(BinWriter& w, const RMSNorm& n) { write(w, n.weight); w.f64(n.eps); w.u64(n.dim); }
inline void read(BinReader& r, RMSNorm* n) { n->weight = read_tensor(r); n->eps = r.f64(); n->dim = (size_t)r.u64(); TALOS_ASSERT(n->weight.len() == n->dim, "RMSNorm weight length does not match dim"); }
inline void write(BinWriter& w, const MLAConfig& c) { for (size_t v : {c.dim, c.num_heads, c.q_lora_rank, c.kv_lora_rank, c.qk_rope_dim, c.v_head_dim, c.max_seq_len}) w.u64(v); }
inline void read(BinReader& r, MLAConfig* c) { for (size_t* v : {&c->dim, &c->num_heads, &c->q_lora_rank, &c->kv_lora_rank, &c->qk_rope_dim, &c->v_head_dim, &c->max_seq_len}) *v = (size_t)r.u64(); }
inline void write(BinWriter& w, const RoPE& r) {
  std::vector<double> c, s; rope_tables_f64(r.dim, r.max_len, r.base, &c, &s);
  w.u64(r.dim); w.f64(r.base); w.vec_f64(c); w.vec_f64(s);
}
inline void read(BinReader& r, RoPE* p) {
  const size_t dim = (size_t)r.u64(); const double base = r.f64();
  const std::vector<double> c = r.vec_f64(), s = r.vec_f64();
  rope_from_tables(p, dim, base, c, s);
}
inline void write(BinWriter& w, const MultiHeadLatentAttention& m) {
  write(w, m.config);
  for (const Linear* l : {&m.w_dkv, &m.w_uk, &m.w_uv, &m.w_q, &m.w_kr, &m.w_qr, &m.w_o}) write(w, *l);
  write(w, m.rope);
}
inline void read(BinReader& r, MultiHeadLatentAttention* m) {
  read(r, &m->config);
  for (Linear* l : {&m->w_dkv, &m->w_uk, &m->w_uv, &m->w_q, &m->w_kr, &m->w_qr, &m->w_o}) read(r, l);
  read(r, &m->rope);
}
inline void write(BinWriter& w, const LuckTransformer& t) {
  write(w, t.embed); write(w, t.norm_1); write(w, t.mla_layer); write(w, t.norm_2); write(w, t.ffn_1); write(w, t.ffn_2); write(w, t.norm_final); write(w, t.out_proj);
}
inline void read(BinReader& r, LuckTransformer* t) {
  read(r, &t->embed); read(r, &t->norm_1); read(r, &t->mla_layer); read(r, &t->norm_2); read(r, &t->ffn_1); read(r, &t->ffn_2); read(r, &t->norm_final); read(r, &t->out_proj);
}
inline void write(BinWriter& w, const ActorCritic& a) { write(w, a.backbone); write(w, a.actor_head); write(w, a.critic_head); }
inline void read(BinReader& r, ActorCritic* a) { read(r, &a->backbone); read(r, &a->actor_head); read(r, &a->critic_head); }

inline std::vector<uint8_t> to_bincode(const ActorCritic& a) { BinWriter w; write(w, a); return std::move(w.buf); }
inline ActorCritic actor_critic_from_bincode(const std::vector<uint8_t>& bytes) {
  ActorCritic a{Uninit{}}; BinReader r(bytes); read(r, &a);
  TALOS_ASSERT(r.o == bytes.size(), "trailing bytes after the model");            // (bincode::deserialize_from itself would stop reading here)
  return a;
}

// ------------------------------------------------------------------ JSON
// An f64 the way serde_json prints it: shortest round-trip digits, laid out by the rules of the `ryu` crate's pretty
// printer.  With the digit string d1..dn and decimal exponent e10 (value = 0.d1..dn x 10^kk, kk = position of the point):
//   n <= kk <= 16      digits, zeros up to the point, ".0"             1234e3 -> 1234000.0
//   0 < kk <= 16       point inside the digits                         12.34
//   -5 < kk <= 0       "0." zeros digits                               0.001234
//   otherwise          d1[.d2..dn]e<exp>, exp = kk - 1, no '+'         1e-6, 1.2345e-7, 1e21
inline std::string fmt_f64(double x) {
  if (!std::isfinite(x)) return "null";
  if (x == 0.0) return std::signbit(x) ? "-0.0" : "0.0";
  char tmp[64];
  auto res = std::to_chars(tmp, tmp + sizeof(tmp), x, std::chars_format::scientific);     // shortest round-trip, d[.ddd]e[+-]xx
  std::string sci(tmp, res.ptr);
  std::string out; size_t i = 0;
  if (sci[0] == '-') { out.push_back('-'); i = 1; }
  const size_t epos = sci.find('e');
  std::string digits;
  for (size_t j = i; j < epos; ++j) if (sci[j] != '.') digits.push_back(sci[j]);
  const int exp10 = std::stoi(sci.substr(epos + 1));
  const int n = (int)digits.size(), kk = exp10 + 1;
  if (n <= kk && kk <= 16) { out += digits; out.append((size_t)(kk - n), '0'); out += ".0"; }
  else if (0 < kk && kk <= 16) { out += digits.substr(0, (size_t)kk); out.push_back('.'); out += digits.substr((size_t)kk); }
  else if (-5 < kk && kk <= 0) { out += "0."; out.append((size_t)(-kk), '0'); out += digits; }
  else { out.push_back(digits[0]); if (n > 1) { out.push_back('.'); out += digits.substr(1); } out.push_back('e'); out += std::to_string(kk - 1); }
  return out;
}

struct JsonWriter {
  std::string s;
  void key(const char* k) { s.push_back('"'); s += k; s += "\":"; }
  void usize(size_t v) { s += std::to_string(v); }
  void f64(double v) { s += fmt_f64(v); }
  void vec_f64(const std::vector<double>& v) { s.push_back('['); for (size_t i = 0; i < v.size(); ++i) { if (i) s.push_back(','); f64(v[i]); } s.push_back(']'); }
  void vec_usize(const std::vector<size_t>& v) { s.push_back('['); for (size_t i = 0; i < v.size(); ++i) { if (i) s.push_back(','); usize(v[i]); } s.push_back(']'); }
};
inline void write(JsonWriter& w, const Tensor& t) { w.s.push_back('{'); w.key("data"); w.vec_f64(t.to_vec()); w.s.push_back(','); w.key("shape"); w.vec_usize(t.shape); w.s.push_back('}'); }
inline void write(JsonWriter& w, const Linear& l) {
  w.s.push_back('{'); w.key("weight"); write(w, l.weight); w.s.push_back(','); w.key("bias");
  if (l.bias) write(w, *l.bias); else w.s += "null";
  w.s.push_back(','); w.key("in_features"); w.usize(l.in_features); w.s.push_back(','); w.key("out_features"); w.usize(l.out_features); w.s.push_back('}');
}
inline void write(JsonWriter& w, const RMSNorm& n) {
  w.s.push_back('{'); w.key("weight"); write(w, n.weight); w.s.push_back(','); w.key("eps"); w.f64(n.eps); w.s.push_back(','); w.key("dim"); w.usize(n.dim); w.s.push_back('}');
}
inline void write(JsonWriter& w, const MLAConfig& c) {
  const char* names[7] = {"dim", "num_heads", "q_lora_rank", "kv_lora_rank", "qk_rope_dim", "v_head_dim", "max_seq_len"};
  const size_t vals[7] = {c.dim, c.num_heads, c.q_lora_rank, c.kv_lora_rank, c.qk_rope_dim, c.v_head_dim, c.max_seq_len};
  w.s.push_back('{'); for (int i = 0; i < 7; ++i) { if (i) w.s.push_back(','); w.key(names[i]); w.usize(vals[i]); } w.s.push_back('}');
}
inline void write(JsonWriter& w, const RoPE& r) {
  std::vector<double> c, s; rope_tables_f64(r.dim, r.max_len, r.base, &c, &s);
  w.s.push_back('{'); w.key("dim"); w.usize(r.dim); w.s.push_back(','); w.key("base"); w.f64(r.base); w.s.push_back(','); w.key("cos_cache"); w.vec_f64(c);
  w.s.push_back(','); w.key("sin_cache"); w.vec_f64(s); w.s.push_back('}');
}
inline void write(JsonWriter& w, const MultiHeadLatentAttention& m) {
  w.s.push_back('{'); w.key("config"); write(w, m.config);
  const char* names[7] = {"w_dkv", "w_uk", "w_uv", "w_q", "w_kr", "w_qr", "w_o"}; const Linear* ls[7] = {&m.w_dkv, &m.w_uk, &m.w_uv, &m.w_q, &m.w_kr, &m.w_qr, &m.w_o};
  for (int i = 0; i < 7; ++i) { w.s.push_back(','); w.key(names[i]); write(w, *ls[i]); }
  w.s.push_back(','); w.key("rope"); write(w, m.rope); w.s.push_back('}');
}
inline void write(JsonWriter& w, const LuckTransformer& t) {
  w.s.push_back('{'); w.key("embed"); write(w, t.embed); w.s.push_back(','); w.key("norm_1"); write(w, t.norm_1); w.s.push_back(','); w.key("mla_layer"); write(w, t.mla_layer);
  w.s.push_back(','); w.key("norm_2"); write(w, t.norm_2); w.s.push_back(','); w.key("ffn_1"); write(w, t.ffn_1); w.s.push_back(','); w.key("ffn_2"); write(w, t.ffn_2);
  w.s.push_back(','); w.key("norm_final"); write(w, t.norm_final); w.s.push_back(','); w.key("out_proj"); write(w, t.out_proj); w.s.push_back('}');
}
inline std::string to_json(const ActorCritic& a) {
  JsonWriter w; w.s.push_back('{'); w.key("backbone"); write(w, a.backbone); w.s.push_back(','); w.key("actor_head"); write(w, a.actor_head);
  w.s.push_back(','); w.key("critic_head"); write(w, a.critic_head); w.s.push_back('}');
  return std::move(w.s);
}

// A reader for exactly this schema.  Like serde's derived Deserialize it takes a struct's keys in any order, ignores
// unknown ones and panics on a missing one; whitespace between tokens is accepted.
struct JsonReader {
  const char* p; const char* end;
  explicit JsonReader(const std::string& s) : p(s.data()), end(s.data() + s.size()) {}
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool peek(char c) { ws(); return p < end && *p == c; }
  void expect(char c) { ws(); TALOS_ASSERT(p < end && *p == c, std::string("model JSON: expected '") + c + "'"); ++p; }
  bool lit(const char* w) { ws(); const size_t n = std::strlen(w); if ((size_t)(end - p) >= n && std::strncmp(p, w, n) == 0) { p += n; return true; } return false; }
  std::string str() { expect('"'); const char* b = p; while (p < end && *p != '"') { TALOS_ASSERT(*p != '\\', "model JSON: escapes are not expected in keys"); ++p; } std::string s(b, p); expect('"'); return s; }
  double num() {
    ws(); TALOS_ASSERT(!lit("null"), "model JSON: null where a number is expected");
    const char* b = p; while (p < end && (std::isdigit((unsigned char)*p) || *p == '-' || *p == '+' || *p == '.' || *p == 'e' || *p == 'E')) ++p;
    TALOS_ASSERT(p > b, "model JSON: number expected");
    return std::strtod(std::string(b, p).c_str(), nullptr);
  }
  size_t usize() { const double v = num(); TALOS_ASSERT(v >= 0 && v == std::floor(v), "model JSON: non-negative integer expected"); return (size_t)v; }
  std::vector<double> vec_f64() { std::vector<double> v; expect('['); if (!peek(']')) { do v.push_back(num()); while (peek(',') && (++p, true)); } expect(']'); return v; }
  std::vector<size_t> vec_usize() { std::vector<size_t> v; expect('['); if (!peek(']')) { do v.push_back(usize()); while (peek(',') && (++p, true)); } expect(']'); return v; }
  void skip_value() {                                             // an unknown key's value
    ws(); TALOS_ASSERT(p < end, "model JSON: truncated");
    if (*p == '{' || *p == '[') { const char open = *p, close = open == '{' ? '}' : ']'; int depth = 0; bool in_str = false;
      for (; p < end; ++p) { if (in_str) { if (*p == '\\') ++p; else if (*p == '"') in_str = false; } else if (*p == '"') in_str = true; else if (*p == open) ++depth; else if (*p == close && --depth == 0) { ++p; return; } }
      TALOS_ASSERT(false, "model JSON: truncated"); }
    if (*p == '"') { str(); return; }
    if (lit("null") || lit("true") || lit("false")) return;
    num();
  }
  // Calls field(key) for every key of the object at the cursor; `field` returns false for a key it does not know.
  template <class F> void object(F&& field) {
    expect('{'); if (peek('}')) { ++p; return; }
    do { const std::string k = str(); expect(':'); if (!field(k)) skip_value(); } while (peek(',') && (++p, true));
    expect('}');
  }
};
inline void require_fields(unsigned seen, unsigned all, const char* what) { TALOS_ASSERT(seen == all, std::string("model JSON: missing field in ") + what); }

inline Tensor read_tensor(JsonReader& r) {
  std::vector<double> data; std::vector<size_t> shape; unsigned seen = 0;
  r.object([&](const std::string& k) { if (k == "data") { data = r.vec_f64(); seen |= 1; } else if (k == "shape") { shape = r.vec_usize(); seen |= 2; } else return false; return true; });
  require_fields(seen, 3, "Tensor"); TALOS_ASSERT(numel(shape) == data.size(), "Data length must match shape");
  return Tensor::new_(data, std::move(shape));
}
inline void read(JsonReader& r, Linear* l) {
  unsigned seen = 0;
  r.object([&](const std::string& k) {
    if (k == "weight") { l->weight = read_tensor(r); seen |= 1; }
    else if (k == "bias") { if (r.lit("null")) l->bias.reset(); else l->bias = read_tensor(r); seen |= 2; }
    else if (k == "in_features") { l->in_features = r.usize(); seen |= 4; }
    else if (k == "out_features") { l->out_features = r.usize(); seen |= 8; }
    else return false;
    return true; });
  require_fields(seen | 2, 15, "Linear");                          // (an absent Option field deserialises as None)
  TALOS_ASSERT(l->weight.shape == (std::vector<size_t>{l->in_features, l->out_features}), "Linear weight shape does not match its feature counts");
}
inline void read(JsonReader& r, RMSNorm* n) {
  unsigned seen = 0;
  r.object([&](const std::string& k) { if (k == "weight") { n->weight = read_tensor(r); seen |= 1; } else if (k == "eps") { n->eps = r.num(); seen |= 2; } else if (k == "dim") { n->dim = r.usize(); seen |= 4; } else return false; return true; });
  require_fields(seen, 7, "RMSNorm"); TALOS_ASSERT(n->weight.len() == n->dim, "RMSNorm weight length does not match dim");
}
inline void read(JsonReader& r, MLAConfig* c) {
  const char* names[7] = {"dim", "num_heads", "q_lora_rank", "kv_lora_rank", "qk_rope_dim", "v_head_dim", "max_seq_len"};
  size_t* vals[7] = {&c->dim, &c->num_heads, &c->q_lora_rank, &c->kv_lora_rank, &c->qk_rope_dim, &c->v_head_dim, &c->max_seq_len};
  unsigned seen = 0;
  r.object([&](const std::string& k) { for (int i = 0; i < 7; ++i) if (k == names[i]) { *vals[i] = r.usize(); seen |= 1u << i; return true; } return false; });
  require_fields(seen, 127, "MLAConfig");
}
inline void read(JsonReader& r, RoPE* p) {
  size_t dim = 0; double base = 0; std::vector<double> c, s; unsigned seen = 0;
  r.object([&](const std::string& k) {
    if (k == "dim") { dim = r.usize(); seen |= 1; } else if (k == "base") { base = r.num(); seen |= 2; }
    else if (k == "cos_cache") { c = r.vec_f64(); seen |= 4; } else if (k == "sin_cache") { s = r.vec_f64(); seen |= 8; } else return false;
    return true; });
  require_fields(seen, 15, "RoPE"); rope_from_tables(p, dim, base, c, s);
}
inline void read(JsonReader& r, MultiHeadLatentAttention* m) {
  const char* names[7] = {"w_dkv", "w_uk", "w_uv", "w_q", "w_kr", "w_qr", "w_o"}; Linear* ls[7] = {&m->w_dkv, &m->w_uk, &m->w_uv, &m->w_q, &m->w_kr, &m->w_qr, &m->w_o};
  unsigned seen = 0;
  r.object([&](const std::string& k) {
    if (k == "config") { read(r, &m->config); seen |= 1u << 7; return true; }
    if (k == "rope") { read(r, &m->rope); seen |= 1u << 8; return true; }
    for (int i = 0; i < 7; ++i) if (k == names[i]) { read(r, ls[i]); seen |= 1u << i; return true; }
    return false; });
  require_fields(seen, 511, "MultiHeadLatentAttention");
}
inline void read(JsonReader& r, LuckTransformer* t) {
  unsigned seen = 0;
  r.object([&](const std::string& k) {
    if (k == "embed") { read(r, &t->embed); seen |= 1; } else if (k == "norm_1") { read(r, &t->norm_1); seen |= 2; } else if (k == "mla_layer") { read(r, &t->mla_layer); seen |= 4; }
    else if (k == "norm_2") { read(r, &t->norm_2); seen |= 8; } else if (k == "ffn_1") { read(r, &t->ffn_1); seen |= 16; } else if (k == "ffn_2") { read(r, &t->ffn_2); seen |= 32; }
    else if (k == "norm_final") { read(r, &t->norm_final); seen |= 64; } else if (k == "out_proj") { read(r, &t->out_proj); seen |= 128; } else return false;
    return true; });
  require_fields(seen, 255, "LuckTransformer");
}
inline ActorCritic actor_critic_from_json(const std::string& text) {
  ActorCritic a{Uninit{}}; JsonReader r(text); unsigned seen = 0;
  r.object([&](const std::string& k) {
    if (k == "backbone") { read(r, &a.backbone); seen |= 1; } else if (k == "actor_head") { read(r, &a.actor_head); seen |= 2; }
    else if (k == "critic_head") { read(r, &a.critic_head); seen |= 4; } else return false;
    return true; });
  require_fields(seen, 7, "ActorCritic");
  return a;
}

// ------------------------------------------------------------------ files (src/main.rs:123-166)
inline bool write_file(const std::string& path, const void* data, size_t n) {
  std::ofstream f(path, std::ios::binary); if (!f) return false;
  f.write((const char*)data, (std::streamsize)n); return (bool)f;
}
inline bool read_file(const std::string& path, std::string* out) {
  std::ifstream f(path, std::ios::binary); if (!f) return false;
  out->assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>()); return true;
}
// Writes `<path>.bin` (bincode) and `<path>` (JSON), as save_ppo_model does.
inline bool save_ppo_model(const ActorCritic& model, const std::string& path) {
  const std::vector<uint8_t> bin = to_bincode(model); const std::string js = to_json(model);
  const bool a = write_file(path + ".bin", bin.data(), bin.size()), b = write_file(path, js.data(), js.size());
  return a && b;
}
// Binary first, JSON as the fallback (also when the binary file does not parse), nothing -> empty optional.
inline std::optional<ActorCritic> load_ppo_model(const std::string& path) {
  std::string raw;
  if (read_file(path + ".bin", &raw)) {
    try { return actor_critic_from_bincode(std::vector<uint8_t>(raw.begin(), raw.end())); } catch (const Panic&) {}
  }
  if (read_file(path, &raw)) {
    try { return actor_critic_from_json(raw); } catch (const Panic&) {}
  }
  return std::nullopt;
}

}  // namespace serde
}  // namespace talos
