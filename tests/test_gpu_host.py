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


def run_driver(args, symmetric=True):
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
