"""The C++ host mirror of the crate's Tensor / autograd / Module API (talos-xii_b200/host/talos.hpp):
the reference's own unit tests replayed through it, and full-model gradients against the oracle."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

import oracle as orc
from oracle import model as om

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp", "bin")


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_reference_unit_tests_through_host_mirror(mode):
    r = subprocess.run([os.path.join(BIN, "test_reference_kats"), str(mode)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0 and "0 failure(s)" in r.stdout, r.stdout


def run_driver32(args):
    with tempfile.NamedTemporaryFile(suffix=".bin") as f:
        r = subprocess.run([os.path.join(BIN, "host_driver")] + [str(a) for a in args[:2]] + [f.name] + [str(a) for a in args[2:]],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1200)
        assert r.returncode == 0, r.stdout
        return np.fromfile(f.name, dtype=np.float32).astype(np.float64)


def run_driver(args, symmetric=True):  # (args after the first two go behind the output file name)
    env = dict(os.environ)
    if symmetric: env["TALOS_SYMMETRIC_WEIGHTS"] = "1"
    with tempfile.NamedTemporaryFile(suffix=".bin") as f:
        r = subprocess.run([os.path.join(BIN, "host_driver")] + [str(a) for a in args[:2]] + [f.name] + [str(a) for a in args[2:]],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
        assert r.returncode == 0, r.stdout
        return np.fromfile(f.name, dtype=np.float64)


def sym(W, fin, fout):
    """w <- 2w + limit: the driver's spread of the half-range LCG stream over [-limit, limit)."""
    return orc.f32r(2.0 * W + np.sqrt(6.0 / (fin + fout)))


def split(flat, shapes):
    out, o = [], 0
    for s in shapes:
        n = int(np.prod(s)); out.append(flat[o:o + n].reshape(s)); o += n
    assert o == flat.size
    return out


@pytest.mark.parametrize("mode,tol", [(0, 2e-5), (1, 2e-5), (2, 4e-3)])
def test_luck_transformer_gradients_match_oracle(mode, tol):
    seed, B, S, fin, hid = 42, 3, 7, 8, 64           # the reference's sizes: 8 features, hidden 64 (src/ppo.rs:255)
    flat = run_driver(["luck", mode, seed, B, S, fin, hid])
    ref = om.LuckTransformer(fin, hid, seed)
    x = orc.f32r(orc.lcg_rand((B, S, fin), -0.5, 0.5, seed + 1000))
    for name in ("embed", "ffn_1", "ffn_2", "out_proj"):      # the device holds fp32 copies of the (spread) LCG weights
        W, b = getattr(ref, name); setattr(ref, name, (sym(W, *W.shape), b))
    ref.mla = {k: sym(v, *v.shape) for k, v in ref.mla.items()}
    g = np.full((B, S, hid), 1.0 / (B * S * hid))
    out, dx, grads = ref.forward_backward(x, g)
    got = split(flat, [out.shape, dx.shape] + [t.shape for t in grads])
    names = ["out", "dx", "embed.W", "embed.b", "norm_1", "dkv", "uk", "uv", "q", "kr", "qr", "o", "norm_2", "ffn1.W", "ffn1.b", "ffn2.W", "ffn2.b", "norm_f", "out.W", "out.b"]
    errs = {}
    for n, a, b in zip(names, got, [out, dx] + grads):
        den = np.linalg.norm(b)
        errs[n] = np.linalg.norm(a - b) / den if den > 0 else np.linalg.norm(a)
    print(mode, {k: "%.1e" % v for k, v in errs.items()})
    for n, e in errs.items():
        assert e <= tol, (n, e)


def test_mla_gradients_match_oracle():
    seed, B, S = 42, 2, 5
    flat = run_driver(["mla", 0, seed, B, S])
    cfg = om.MLAConfig(16, 2, 8, 4, 8, 64)
    W = {k: sym(v, *v.shape) for k, v in om.mla_init_lcg(cfg, seed).items()}
    x = orc.f32r(orc.lcg_rand((B, S, 16), -0.5, 0.5, seed + 1000))
    out, cache = om.mla_forward(x, W, cfg, "head_index", return_cache=True)
    dx, dW = om.mla_backward(np.full(out.shape, 1.0 / out.size), W, cfg, cache, "head_index")
    ref = [out, dx] + [dW[k] for k in ("dkv", "uk", "uv", "q", "kr", "qr", "o")]
    got = split(flat, [t.shape for t in ref])
    for a, b in zip(got, ref):
        assert np.linalg.norm(a - b) <= 2e-5 * np.linalg.norm(b)


def nrm(seed, shape, std=1.0):
    return orc.f32r(orc.rng_normal(seed, shape, 0.0, 1.0) * np.float64(np.float32(std))) if False else orc.rng_normal(seed, shape, 0.0, std).astype(np.float32).astype(np.float64)


@pytest.mark.parametrize("mode,tol", [(1, 1e-5), (2, 2e-3)])
def test_config3_transformer_block_forward_backward(mode, tol):
    # benchmark configuration 3 shapes (S64 d256 H8 dh32 ff1024, eps 1e-6, RoPE base 10000 token positions, causal, SiLU);
    # the oracle runs a 32-sample batch, the GPU also the full 1024-sample batch.
    Bs, S, D, H = 32, 64, 256, 8
    P = dict(g1=np.ones(D), g2=np.ones(D), w_qkv=nrm(11, (D, 3 * D), 0.02), w_o=nrm(12, (D, D), 0.02), w_ff1=nrm(13, (D, 1024), 0.02),
             w_ff2=nrm(14, (1024, D), 0.02))
    x = nrm(10, (Bs, S, D)); G = nrm(15, (Bs, S, D))
    # the block lays QKV out as [q | k | v] per token; the oracle block as [3, H, dh] per token: same thing
    y, cache = om.block_fwd(x, P, H, eps=1e-6)
    dx, dP = om.block_bwd(G, P, cache)
    flat = run_driver32(["block", mode, Bs, Bs, 0])
    ref = [y, dx, dP["g1"], dP["w_qkv"], dP["w_o"], dP["g2"], dP["w_ff1"], dP["w_ff2"]]
    got = split(flat, [t.shape for t in ref])
    for n, a, b in zip(["out", "dx", "dg1", "dWqkv", "dWo", "dg2", "dWff1", "dWff2"], got, ref):
        err = np.linalg.norm(a - b) / np.linalg.norm(b)
        assert err <= 2 * tol, (n, err)          # fp32 dump of the result adds up to 6e-8; gradients chain ~10 GEMMs
    if mode == 1:
        # full configuration (batch 1024): samples are independent, so its first 32 samples must reproduce the small run
        full = run_driver32(["block", mode, Bs, 1024, 0])
        gf = split(full, [t.shape for t in ref])
        assert np.linalg.norm(gf[0] - got[0]) <= tol * np.linalg.norm(got[0])
        assert np.linalg.norm(gf[1] - got[1]) <= tol * np.linalg.norm(got[1])
        assert np.all(np.isfinite(full))


@pytest.mark.parametrize("mode,tol", [(1, 1e-5), (2, 2e-3)])
def test_config4_mla_forward_both_position_modes(mode, tol):
    # benchmark configuration 4 shapes: S128 d512 latent 64, 8 heads of 64 + rope 32, N(0,0.02^2) weights, non-causal
    Bs, S, D = 16, 128, 512
    cfg = om.MLAConfig(D, 8, 64, 32, 64, 128)
    shapes = dict(dkv=(D, 64), uk=(64, 512), uv=(64, 512), q=(D, 512), kr=(D, 256), qr=(D, 256), o=(512, D))
    W = {k: nrm(21 + i, shapes[k], 0.02) for i, k in enumerate(["dkv", "uk", "uv", "q", "kr", "qr", "o"])}
    x = nrm(20, (Bs, S, D))
    outs = {}
    for token in (1, 0):
        ref = om.mla_forward(x, W, cfg, "token" if token else "head_index")
        got = run_driver32(["mla4", mode, Bs, Bs, token]).reshape(ref.shape)
        err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert err <= tol, (token, err)
        outs[token] = got
    assert np.linalg.norm(outs[0] - outs[1]) > 1e-3 * np.linalg.norm(outs[1])    # the two conventions really differ here
    if mode == 1:
        full = run_driver32(["mla4", mode, Bs, 512, 1]).reshape(outs[1].shape)    # full batch 512: first samples unchanged
        # (tile shapes and split-K differ with the batch size, so agreement is to the mode's tolerance, not bit-exact)
        assert np.linalg.norm(full - outs[1]) <= tol * np.linalg.norm(outs[1])


@pytest.mark.parametrize("mode,tol", [(1, 1e-5), (2, 2e-3)])
def test_config3_full_batch_interior_samples_against_the_oracle(mode, tol):
    # benchmark configuration 3 at its full batch of 1024: samples are independent given the weights, so the oracle
    # runs 32 samples from the MIDDLE of the batch (rows 500..531 of the same seeded input) and the device's output
    # and input gradient for exactly those samples must match
    Bf, Bs, start, S, D, H = 1024, 32, 500, 64, 256, 8
    P = dict(g1=np.ones(D), g2=np.ones(D), w_qkv=nrm(11, (D, 3 * D), 0.02), w_o=nrm(12, (D, D), 0.02), w_ff1=nrm(13, (D, 1024), 0.02),
             w_ff2=nrm(14, (1024, D), 0.02))
    x = nrm(10, (Bf, S, D))[start:start + Bs]; G = nrm(15, (Bf, S, D))[start:start + Bs]
    y, cache = om.block_fwd(x, P, H, eps=1e-6)
    dx, _ = om.block_bwd(G, P, cache)
    flat = run_driver32(["block", mode, Bs, Bf, 0, start])
    got_y, got_dx = split(flat[:2 * Bs * S * D], [y.shape, dx.shape])
    assert np.all(np.isfinite(flat))
    for n, a, b in (("out", got_y, y), ("dx", got_dx, dx)):
        err = np.linalg.norm(a - b) / np.linalg.norm(b)
        assert err <= 2 * tol, (n, err)


@pytest.mark.parametrize("mode,tol", [(1, 1e-5), (2, 2e-3)])
def test_config4_full_batch_interior_samples_against_the_oracle(mode, tol):
    # benchmark configuration 4 at its full batch of 512, token positions: samples 240..271 against the oracle
    Bf, Bs, start, S, D = 512, 32, 240, 128, 512
    cfg = om.MLAConfig(D, 8, 64, 32, 64, 128)
    shapes = dict(dkv=(D, 64), uk=(64, 512), uv=(64, 512), q=(D, 512), kr=(D, 256), qr=(D, 256), o=(512, D))
    W = {k: nrm(21 + i, shapes[k], 0.02) for i, k in enumerate(["dkv", "uk", "uv", "q", "kr", "qr", "o"])}
    x = nrm(20, (Bf, S, D))[start:start + Bs]
    ref = om.mla_forward(x, W, cfg, "token")
    got = run_driver32(["mla4", mode, Bs, Bf, 1, start]).reshape(ref.shape)
    err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert err <= tol, err


@pytest.mark.parametrize("mode,tol", [(0, 1e-5), (1, 1e-5), (2, 2e-3)])
def test_batched_rollout_matches_per_simulation_cached_inference(mode, tol):
    # ActorCritic::step_inference_cached (src/ppo.rs:391-432) + prune_cache (src/sim.rs:171-175) per simulation in the
    # oracle vs. one batched step over all simulations on the device.  23 steps with a context of 6 make every ring
    # wrap several times; the reset pattern leaves the simulations at different positions; N = 37 is not a multiple
    # of the kernel's 8 warps per block.
    seed, N, T, ctx = 42, 37, 23, 6
    got = run_driver(["rollout", mode, seed, N, T, ctx]).reshape(T, N, 5)
    ac = om.ActorCritic(seed)
    bb = ac.backbone
    for name in ("embed", "ffn_1", "ffn_2", "out_proj"):
        W, b = getattr(bb, name); setattr(bb, name, (sym(W, *W.shape), b))
    bb.mla = {k: sym(v, *v.shape) for k, v in bb.mla.items()}
    ac.actor = (sym(ac.actor[0], *ac.actor[0].shape), ac.actor[1])
    states = nrm(seed + 500, (T, N, 8), 0.5)
    resets = np.array([[1 if (t * 7 + n * 3) % 11 == 0 else 0 for n in range(N)] for t in range(T)])
    ref = om.rollout_reference(ac, states, resets, ctx)
    err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert err <= tol, err
    assert np.abs(got.sum(-1) - 1.0).max() < 1e-5
    if mode != 2:   # identical argmax wherever the oracle's top two probabilities are not within rounding of each other
        top2 = np.sort(ref, -1)[..., -2:]
        clear = (top2[..., 1] - top2[..., 0]) > 1e-4
        assert np.array_equal(got.argmax(-1)[clear], ref.argmax(-1)[clear])


def test_batched_rollout_with_the_crates_own_weights():
    # the same comparison with the crate's own initialisation left as it is (half-range LCG: every weight negative),
    # the reference's sizes (8 features, hidden 64, 5 actions), context 3, 5 simulations x 9 steps
    seed, N, T, ctx_len = 7, 5, 9, 3
    got = run_driver(["rollout", 1, seed, N, T, ctx_len], symmetric=False).reshape(T, N, 5)
    states = nrm(seed + 500, (T, N, 8), 0.5)
    resets = np.array([[1 if (t * 7 + n * 3) % 11 == 0 else 0 for n in range(N)] for t in range(T)])
    ref = om.rollout_reference(om.ActorCritic(seed), states, resets, ctx_len)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-5


def _ryu_like(x):
    """An f64 as serde_json writes it: shortest round-trip digits in the layout of the `ryu` crate (see
    talos-xii_b200/host/talos_serde.hpp), written independently here from Python's own shortest-digits repr."""
    import math
    if not math.isfinite(x):
        return "null"
    if x == 0.0:
        return "-0.0" if math.copysign(1.0, x) < 0 else "0.0"
    sign = "-" if x < 0 else ""
    m, e = ("%r" % abs(x)).lower(), 0
    if "e" in m:
        m, ee = m.split("e"); e = int(ee)
    ip, _, fp = m.partition(".")
    digits = (ip + fp).lstrip("0"); kk = len(ip.lstrip("0")) + e if ip.strip("0") else e - (len(fp) - len(fp.lstrip("0")))
    digits = digits.rstrip("0") or "0"; n = len(digits)
    if n <= kk <= 16:
        return sign + digits + "0" * (kk - n) + ".0"
    if 0 < kk <= 16:
        return sign + digits[:kk] + "." + digits[kk:]
    if -5 < kk <= 0:
        return sign + "0." + "0" * (-kk) + digits
    return sign + digits[0] + ("." + digits[1:] if n > 1 else "") + "e" + str(kk - 1)


def test_ryu_like_formatter_known_cases():
    # (the fixed-point form reaches down to four zeros after the point: 1e-5 is 0.00001, 1e-6 is 1e-6)
    cases = {1.0: "1.0", 10000.0: "10000.0", 1e-5: "0.00001", 1e-6: "1e-6", 0.001: "0.001", 1.2345e-7: "1.2345e-7", 1e16: "1e16", 1e15: "1000000000000000.0",
             -0.5: "-0.5", 123456.789: "123456.789", 1e21: "1e21", 0.00001234: "0.00001234", 1.234e-6: "1.234e-6", 1234000.0: "1234000.0",
             float(np.float32(0.1)): "0.10000000149011612"}
    for v, want in cases.items():
        assert _ryu_like(v) == want, (v, _ryu_like(v), want)


def test_model_files_have_the_crates_byte_layout_and_round_trip(tmp_path):
    # save_ppo_model / load_ppo_model (src/main.rs:123-166): the files the host mirror writes are compared, byte for
    # byte, with files assembled here by hand from the bincode 1.x / serde_json rules and the oracle's copy of the
    # LCG-initialised weights; the models read back from them must compute exactly what the original computes.
    import math
    import struct
    seed, B, S = 12345, 2, 3
    prefix = str(tmp_path / "ppo.cache")
    flat = run_driver(["serde", 0, seed, B, S, prefix], symmetric=False)
    outs = flat.reshape(5, -1)
    for i in range(1, 5):
        assert np.array_equal(outs[0], outs[i]), i
    ac = om.ActorCritic(seed)
    bb = ac.backbone; cfg = bb.cfg
    f32 = lambda a: np.asarray(a, dtype=np.float64).astype(np.float32).astype(np.float64)
    u64 = lambda v: struct.pack("<Q", v)

    def tensor(a, shape):
        a = f32(a).ravel()
        return u64(a.size) + a.astype("<f8").tobytes() + u64(len(shape)) + b"".join(u64(d) for d in shape)

    def linear(W, b):
        fi, fo = W.shape
        return tensor(W, (fi, fo)) + (b"\x01" + tensor(b, (fo,)) if b is not None else b"\x00") + u64(fi) + u64(fo)

    def rmsnorm(g, eps):
        return tensor(g, (g.size,)) + struct.pack("<d", eps) + u64(g.size)
    cos_t, sin_t = [], []
    dr = cfg.qk_rope_dim
    for pos in range(cfg.max_seq_len):
        for i in range(dr // 2):
            theta = 1.0 / math.pow(10000.0, (2 * i) / dr); ang = pos * theta
            cos_t.append(math.cos(ang)); sin_t.append(math.sin(ang))
    vec = lambda v: u64(len(v)) + np.asarray(v, dtype="<f8").tobytes()
    mla = b"".join(u64(v) for v in (cfg.dim, cfg.num_heads, 0, cfg.kv_lora_rank, cfg.qk_rope_dim, cfg.v_head_dim, cfg.max_seq_len))
    mla += b"".join(linear(bb.mla[k], None) for k in ("dkv", "uk", "uv", "q", "kr", "qr", "o"))
    mla += u64(dr) + struct.pack("<d", 10000.0) + vec(cos_t) + vec(sin_t)
    want = (linear(*bb.embed) + rmsnorm(bb.g1, 1e-5) + mla + rmsnorm(bb.g2, 1e-5) + linear(*bb.ffn_1) + linear(*bb.ffn_2) + rmsnorm(bb.gf, 1e-5)
            + linear(*bb.out_proj) + linear(*ac.actor) + linear(*ac.critic))
    got = open(prefix + ".bin", "rb").read()
    assert len(got) == len(want) and got == want

    # JSON: same content, keys in declaration order, numbers in serde_json's spelling
    num = _ryu_like
    arr = lambda v: "[" + ",".join(num(float(x)) for x in v) + "]"
    jt = lambda a, shape: '{"data":%s,"shape":[%s]}' % (arr(f32(a).ravel()), ",".join(str(d) for d in shape))
    jl = lambda W, b: '{"weight":%s,"bias":%s,"in_features":%d,"out_features":%d}' % (jt(W, W.shape), jt(b, (W.shape[1],)) if b is not None else "null", W.shape[0], W.shape[1])
    jn = lambda g, eps: '{"weight":%s,"eps":%s,"dim":%d}' % (jt(g, (g.size,)), num(eps), g.size)
    jc = '{"dim":%d,"num_heads":%d,"q_lora_rank":0,"kv_lora_rank":%d,"qk_rope_dim":%d,"v_head_dim":%d,"max_seq_len":%d}' % (
        cfg.dim, cfg.num_heads, cfg.kv_lora_rank, cfg.qk_rope_dim, cfg.v_head_dim, cfg.max_seq_len)
    jm = '{"config":%s,%s,"rope":{"dim":%d,"base":10000.0,"cos_cache":%s,"sin_cache":%s}}' % (
        jc, ",".join('"w_%s":%s' % (k, jl(bb.mla[k], None)) for k in ("dkv", "uk", "uv", "q", "kr", "qr", "o")), dr, arr(cos_t), arr(sin_t))
    jb = '{"embed":%s,"norm_1":%s,"mla_layer":%s,"norm_2":%s,"ffn_1":%s,"ffn_2":%s,"norm_final":%s,"out_proj":%s}' % (
        jl(*bb.embed), jn(bb.g1, 1e-5), jm, jn(bb.g2, 1e-5), jl(*bb.ffn_1), jl(*bb.ffn_2), jn(bb.gf, 1e-5), jl(*bb.out_proj))
    want_js = '{"backbone":%s,"actor_head":%s,"critic_head":%s}' % (jb, jl(*ac.actor), jl(*ac.critic))
    got_js = open(prefix).read()
    assert got_js == want_js
    import json
    parsed = json.loads(got_js)                                    # and it is JSON: key order as the structs declare their fields
    assert list(parsed) == ["backbone", "actor_head", "critic_head"]
    assert list(parsed["backbone"]) == ["embed", "norm_1", "mla_layer", "norm_2", "ffn_1", "ffn_2", "norm_final", "out_proj"]
    assert list(parsed["backbone"]["mla_layer"]) == ["config", "w_dkv", "w_uk", "w_uv", "w_q", "w_kr", "w_qr", "w_o", "rope"]
    # the loaded models agree with the oracle's forward on the same LCG states
    x = orc.f32r(orc.lcg_rand((B, S, 8), -0.5, 0.5, seed + 1000))
    for name in ("embed", "ffn_1", "ffn_2", "out_proj"):
        W, b = getattr(bb, name); setattr(bb, name, (f32(W), b))
    bb.mla = {k: f32(v) for k, v in bb.mla.items()}
    ac.actor = (f32(ac.actor[0]), ac.actor[1])
    ref = np.stack([ac.forward_actor(x[i:i + 1]) for i in range(B)]).ravel()
    assert np.linalg.norm(outs[0] - ref) <= 2e-5 * np.linalg.norm(ref)
