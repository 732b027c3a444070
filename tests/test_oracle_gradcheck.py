"""Central-difference checks of the oracle's backward passes.  The reference pins these ops
only with "gradient is non-zero" tests, so finite differences are the authority here
(same method as src/grad_check.rs:93-114: eps 1e-6, tol 1e-4, tightened where f64 allows)."""
import math

import numpy as np

import oracle as orc
from oracle import model as om


def num_grad(f, x, eps=1e-6):
    g = np.zeros_like(x); it = np.nditer(x, flags=["multi_index"])
    for _ in it:
        i = it.multi_index; old = x[i]
        x[i] = old + eps; fp = f()
        x[i] = old - eps; fm = f()
        x[i] = old; g[i] = (fp - fm) / (2 * eps)
    return g


def test_numerical_gradient_check():
    # src/grad_check.rs:93-114: f(x) = x^2 sin x at 2.0
    x = 2.0
    auto = 2 * x * math.sin(x) + x * x * math.cos(x)
    f = lambda v: v * v * math.sin(v)
    assert abs(auto - (f(x + 1e-6) - f(x - 1e-6)) / 2e-6) < 1e-4


def test_rmsnorm_grad():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 8)); w = rng.standard_normal(8); gy = rng.standard_normal((5, 8))
    y, rms, xh = orc.rmsnorm_fwd(x, w, 1e-5)
    assert np.allclose(y, x / np.sqrt((x * x).mean(1, keepdims=True) + 1e-5) * w)
    dx, dw = orc.rmsnorm_bwd(gy, w, rms, xh)
    f = lambda: float((orc.rmsnorm_fwd(x, w, 1e-5)[0] * gy).sum())
    assert np.allclose(dx, num_grad(f, x), atol=1e-6)
    assert np.allclose(dw, num_grad(f, w), atol=1e-6)


def test_rope_grad_and_conventions():
    rng = np.random.default_rng(1)
    cosv, sinv = orc.rope_table(8, 16)
    x = rng.standard_normal((2, 5, 3, 8)); g = rng.standard_normal(x.shape)
    f = lambda: float((orc.rope(x, cosv, sinv, 0) * g).sum())
    assert np.allclose(orc.rope(g, cosv, sinv, 0, backward=True), num_grad(f, x), atol=1e-6)
    # head-index convention: every token gets the same rotation, so q.k per head is what it
    # was before the rotation (rotations preserve inner products)
    r = orc.rope(x, cosv, sinv, 0)
    assert np.allclose(np.einsum("bshd,bthd->bhst", r, r), np.einsum("bshd,bthd->bhst", x, x))
    # token convention differs from it and matches an explicit per-token rotation
    t = orc.rope_token(x, cosv, sinv, 0)
    assert not np.allclose(t, r)
    h = 4
    for s in range(5):
        c = cosv[s * h:(s + 1) * h]; sn = sinv[s * h:(s + 1) * h]
        assert np.allclose(t[:, s, :, 0::2], x[:, s, :, 0::2] * c - x[:, s, :, 1::2] * sn)
        assert np.allclose(t[:, s, :, 1::2], x[:, s, :, 0::2] * sn + x[:, s, :, 1::2] * c)
    # start_pos offsets the table row
    assert np.allclose(orc.rope_token(x[:, :1], cosv, sinv, 3), t[:, 3:4] * 0 + orc.rope_token(np.repeat(x[:, :1], 4, 1), cosv, sinv, 0)[:, 3:4])


def test_softmax_and_bmm_grads():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((3, 4, 4)); g = rng.standard_normal(x.shape)
    y = orc.softmax(x)
    assert np.allclose(y.sum(-1), 1.0)
    f = lambda: float((orc.softmax(x) * g).sum())
    assert np.allclose(orc.softmax_bwd(y, g), num_grad(f, x), atol=1e-6)
    yc = orc.softmax(x, causal_period=4)
    assert np.all(np.triu(yc[0], 1) == 0.0) and np.allclose(yc.sum(-1), 1.0)
    q = rng.standard_normal((3, 4, 6)); k = rng.standard_normal((3, 4, 6)); v = rng.standard_normal((3, 4, 5))
    assert np.allclose(orc.bmm_qkt(q, k), np.einsum("bid,bjd->bij", q, k))
    dq, dk = orc.bmm_qkt_bwd(q, k, g)
    assert np.allclose(dq, np.einsum("bij,bjd->bid", g, k)) and np.allclose(dk, np.einsum("bij,bid->bjd", g, q))
    p = orc.softmax(x); go = rng.standard_normal((3, 4, 5))
    assert np.allclose(orc.bmm_pv(p, v), p @ v)
    dp, dv = orc.bmm_pv_bwd(p, v, go)
    assert np.allclose(dp, go @ v.swapaxes(1, 2)) and np.allclose(dv, p.swapaxes(1, 2) @ go)


def test_mla_grad_both_pos_modes():
    rng = np.random.default_rng(3)
    cfg = om.MLAConfig(8, 2, 4, 4, 4, 8)
    W = {k: 0.3 * rng.standard_normal(v.shape) for k, v in om.mla_init_lcg(cfg, 1).items()}
    x = rng.standard_normal((2, 3, 8)); g = rng.standard_normal((2, 3, 8))
    for mode in ("head_index", "token"):
        out, cache = om.mla_forward(x, W, cfg, mode, return_cache=True)
        dx, dW = om.mla_backward(g, W, cfg, cache, mode)
        f = lambda: float((om.mla_forward(x, W, cfg, mode) * g).sum())
        assert np.allclose(dx, num_grad(f, x), atol=1e-6), mode
        for name in W:
            assert np.allclose(dW[name], num_grad(f, W[name]), atol=1e-6), (mode, name)
    a = om.mla_forward(x, W, cfg, "head_index"); b = om.mla_forward(x, W, cfg, "token")
    assert not np.allclose(a, b)      # with ordinary weights the two conventions give different outputs


def test_block_grad():
    rng = np.random.default_rng(4)
    D, H = 8, 2
    P = dict(g1=1 + 0.1 * rng.standard_normal(D), g2=1 + 0.1 * rng.standard_normal(D),
             w_qkv=0.3 * rng.standard_normal((D, 3 * D)), w_o=0.3 * rng.standard_normal((D, D)),
             w_ff1=0.3 * rng.standard_normal((D, 4 * D)), w_ff2=0.3 * rng.standard_normal((4 * D, D)))
    x = rng.standard_normal((2, 4, D)); g = rng.standard_normal(x.shape)
    y, cache = om.block_fwd(x, P, H)
    dx, dP = om.block_bwd(g, P, cache)
    f = lambda: float((om.block_fwd(x, P, H)[0] * g).sum())
    assert np.allclose(dx, num_grad(f, x), atol=1e-6)
    for name in P:
        assert np.allclose(dP[name], num_grad(f, P[name]), atol=1e-6), name
    # causal: output at token t does not depend on later tokens
    x2 = x.copy(); x2[:, 3] += 1.0
    assert np.allclose(om.block_fwd(x2, P, H)[0][:, :3], y[:, :3])


def test_mlp_grad_all_activations():
    rng = np.random.default_rng(5)
    X = rng.standard_normal((6, 5)); dY = rng.standard_normal((6, 3))
    for act in ("relu", "tanh", "silu"):
        Ws = [0.5 * rng.standard_normal(s) for s in [(5, 7), (7, 7), (7, 3)]]
        bs = [0.1 * rng.standard_normal(s[1]) for s in [(5, 7), (7, 7), (7, 3)]]
        acts = [act, act, "none"]
        zs, hs = om.mlp_fwd(X, Ws, bs, acts)
        dX, dWs, dbs = om.mlp_bwd(X, Ws, bs, acts, zs, hs, dY)
        f = lambda: float((om.mlp_fwd(X, Ws, bs, acts)[1][-1] * dY).sum())
        assert np.allclose(dX, num_grad(f, X), atol=1e-5), act
        for l in range(3):
            assert np.allclose(dWs[l], num_grad(f, Ws[l]), atol=1e-5), (act, l)
            assert np.allclose(dbs[l], num_grad(f, bs[l]), atol=1e-5), (act, l)


def test_ppo_loss_grad_and_branches():
    rng = np.random.default_rng(6)
    n, A = 64, 5
    logits = rng.standard_normal((n, A)); values = rng.standard_normal(n)
    actions = rng.integers(0, A, n); adv = rng.standard_normal(n); ret = rng.standard_normal(n)
    old = rng.standard_normal(n) * 0.3 - 1.6          # spreads ratios on both sides of the clip range
    loss, dl, dv, kl = om.ppo_loss_fwd_bwd(logits, values, actions, old, adv, ret)
    f = lambda: om.ppo_loss_fwd_bwd(logits, values, actions, old, adv, ret)[0]
    assert np.allclose(dl, num_grad(f, logits), atol=1e-7)
    assert np.allclose(dv, num_grad(f, values), atol=1e-7)
    # scalar restatement of src/ppo.rs:702-755 for one sample at a time
    tot = 0.0; kls = 0.0
    for i in range(n):
        mx = logits[i].max(); lse = math.log(np.exp(logits[i] - mx).sum()) + mx
        lp = logits[i] - lse; lr = lp[actions[i]] - old[i]; r = math.exp(lr)
        kls += (r - 1.0) - lr
        s1 = r * adv[i]; s2 = min(max(r, 0.8), 1.2) * adv[i]
        pol = s1 if s1 < s2 else s2
        ent = -(np.exp(lp) * lp).sum()
        tot += -pol + 0.5 * (values[i] - ret[i]) ** 2 - 0.01 * ent
    assert abs(loss - tot / n) < 1e-12 and abs(kl - kls) < 1e-10
    ratio = np.exp(np.log(np.exp(logits - logits.max(1, keepdims=True)) / np.exp(logits - logits.max(1, keepdims=True)).sum(1, keepdims=True))[np.arange(n), actions] - old)
    assert (ratio < 0.8).any() and (ratio > 1.2).any() and ((ratio > 0.8) & (ratio < 1.2)).any()


def test_adam_matches_closed_form_first_step():
    # src/ppo.rs:519-533: after one step from m=v=0, update = lr * g/(|g| + eps)
    p = [np.array([1.0, -2.0, 3.0])]; g = [np.array([0.5, -0.25, 0.0])]
    m = [np.zeros(3)]; v = [np.zeros(3)]
    om.adam_step(p, g, m, v, 1, 3e-4)
    exp = np.array([1.0, -2.0, 3.0]) - 3e-4 * g[0] / (np.abs(g[0]) + 1e-8)
    assert np.allclose(p[0], exp, atol=1e-12)
    # DQN variant: global-norm clip to 1.0 (src/dqn.rs:209-222)
    p2 = [np.zeros(2)]; m2 = [np.zeros(2)]; v2 = [np.zeros(2)]
    om.adam_step(p2, [np.array([3.0, 4.0])], m2, v2, 1, 1e-3, clip_norm=1.0)
    assert np.allclose(m2[0], 0.1 * np.array([0.6, 0.8]))


def test_ppo_update_reduces_loss_and_kl_reporting():
    rng = np.random.default_rng(7)
    n, obs_dim, h, A = 256, 6, 8, 4
    params = dict(w1=0.3 * rng.standard_normal((obs_dim, h)), b1=np.zeros(h), w2=0.3 * rng.standard_normal((h, h)),
                  b2=np.zeros(h), wp=0.3 * rng.standard_normal((h, A)), bp=np.zeros(A),
                  wv=0.3 * rng.standard_normal((h, 1)), bv=np.zeros(1))
    model = om.MlpActorCritic(params)
    obs = rng.standard_normal((n, obs_dim)); actions = rng.integers(0, A, n)
    adv = rng.standard_normal(n); ret = rng.standard_normal(n)
    old = model.log_prob(obs, actions)
    _, l0, kl0 = model.grads(obs, actions, old, adv, ret)
    assert abs(kl0) < 1e-12                      # ratio == 1 at the rollout weights
    kls, opt = om.ppo_update(model, obs, actions, old, adv, ret, epochs=4, minibatch=64, lr=3e-3)
    _, l1, _ = model.grads(obs, actions, old, adv, ret)
    assert l1 < l0 and opt["t"] == 16 and len(kls) == 4 and kls[-1] > 0.0
    # full-batch gradient == sum of minibatch gradients scaled to a common denominator
    g_full, _, _ = model.grads(obs, actions, old, adv, ret)
    acc = {k: 0.0 for k in model.NAMES}
    for s in range(0, n, 64):
        g, _, _ = model.grads(obs[s:s + 64], actions[s:s + 64], old[s:s + 64], adv[s:s + 64], ret[s:s + 64], denom=n)
        for k in acc: acc[k] = acc[k] + g[k]
    for k in acc:
        assert np.allclose(acc[k], g_full[k], atol=1e-12), k
