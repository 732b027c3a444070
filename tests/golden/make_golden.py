"""Generates tests/golden/golden.npz: small seeded inputs and the oracle's f64 outputs for every op of the path.

    python tests/golden/make_golden.py

The reference crate cannot be run here (Rust, no toolchain), so these vectors come from the CPU oracle after it
has been pinned against the crate's own known-answer tests (tests/test_oracle_kat.py); the crate's KAT constants
themselves are included verbatim under the `kat_` keys.  The GPU tests compare the CUDA path with these files, so
a later change to the oracle cannot silently move the target."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as orc                      # noqa: E402
from oracle import model as om           # noqa: E402


def n(seed, shape, std=1.0):
    return orc.f32r(orc.rng_normal(seed, shape, 0.0, std))


def build():
    g = {}
    # known answers of the reference's tests
    g["kat_matmul_A"] = np.array([[2.0, 3.0], [4.0, 5.0]]); g["kat_matmul_x"] = np.array([[1.0], [2.0]])
    g["kat_matmul_y"] = np.array([8.0, 14.0]); g["kat_matmul_dx"] = np.array([6.0, 8.0]); g["kat_matmul_dA"] = np.array([1.0, 2.0, 1.0, 2.0])   # src/grad_check.rs:30-63
    g["kat_transpose_in"] = np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]); g["kat_transpose_out"] = np.array([1.0, 4.0, 2.0, 5.0, 3.0, 6.0])          # src/transformer.rs:1212-1225
    # matmul, three forms
    A = n(1, (17, 13)); B = n(2, (13, 9)); G = n(3, (17, 9))
    g["mm_A"], g["mm_B"], g["mm_G"] = A, B, G
    g["mm_C"] = orc.matmul(A, B); g["mm_dA"], g["mm_dB"] = orc.matmul_bwd(A, B, G)
    # MLP forward/backward (tanh)
    X = n(4, (33, 8)); Ws = [n(5 + i, s, 0.4) for i, s in enumerate([(8, 16), (16, 16), (16, 5)])]; bs = [n(9 + i, (s,), 0.1) for i, s in enumerate([16, 16, 5])]
    dY = n(12, (33, 5)); acts = ["tanh", "tanh", "none"]
    zs, hs = om.mlp_fwd(X, Ws, bs, acts); dX, dWs, dbs = om.mlp_bwd(X, Ws, bs, acts, zs, hs, dY)
    g.update(mlp_X=X, mlp_dY=dY, mlp_Y=hs[-1], mlp_dX=dX)
    for i in range(3):
        g["mlp_W%d" % i], g["mlp_b%d" % i], g["mlp_dW%d" % i], g["mlp_db%d" % i] = Ws[i], bs[i], dWs[i], dbs[i]
    # RMSNorm
    x = n(13, (19, 24)); gam = 1.0 + n(14, (24,), 0.1); gy = n(15, (19, 24))
    y, rms, xh = orc.rmsnorm_fwd(x, gam, 1e-5); dx, dw = orc.rmsnorm_bwd(gy, gam, rms, xh)
    g.update(rms_x=x, rms_gamma=gam, rms_gy=gy, rms_y=y, rms_dx=dx, rms_dgamma=dw)
    # RoPE, both conventions
    cosv, sinv = orc.rope_table(8, 16); cosf, sinf = orc.f32r(cosv), orc.f32r(sinv)
    xr = n(16, (2, 5, 3, 8))
    g.update(rope_x=xr, rope_token=orc.rope_token(xr, cosf, sinf, 2), rope_head=orc.rope(xr, cosf, sinf, 0), rope_head_bwd=orc.rope(xr, cosf, sinf, 0, backward=True))
    # softmax and attention
    s = n(17, (11, 20), 2.0); gs = n(18, (11, 20))
    ys = orc.softmax(s); g.update(sm_x=s, sm_g=gs, sm_y=ys, sm_dx=orc.softmax_bwd(ys, gs), sm_causal=orc.softmax(n(17, (12, 4), 2.0), 4))
    q = n(19, (3, 10, 12)); k = n(20, (3, 10, 12)); v = n(21, (3, 10, 6)); go = n(22, (3, 10, 6)); sc = np.float64(np.float32(1.0 / np.sqrt(12.0)))
    P = orc.softmax(orc.bmm_qkt(q, k) * sc); O = orc.bmm_pv(P, v)
    dP, dv = orc.bmm_pv_bwd(P, v, go); dS = orc.softmax_bwd(P, dP) * sc; dq, dk = orc.bmm_qkt_bwd(q, k, dS)
    g.update(att_q=q, att_k=k, att_v=v, att_go=go, att_P=P, att_O=O, att_dq=dq, att_dk=dk, att_dv=dv)
    # MLA forward, both conventions (reference-shaped: dim16/h2/r8/rope4/dv8)
    cfg = om.MLAConfig(16, 2, 8, 4, 8, 32)
    W = {kk: n(30 + i, vv.shape, 0.3) for i, (kk, vv) in enumerate(om.mla_init_lcg(cfg, 1).items())}
    xm = n(40, (2, 6, 16))
    for kk, vv in W.items(): g["mla_W_" + kk] = vv
    g.update(mla_x=xm, mla_head=om.mla_forward(xm, W, cfg, "head_index"), mla_token=om.mla_forward(xm, W, cfg, "token"))
    # PPO loss and Adam
    lg = n(41, (50, 5)); vl = n(42, (50,)); ac = orc.rng_bounded(43, 50, 5); ad = n(44, (50,)); rt = n(45, (50,)); ol = orc.f32r(-1.6 + 0.4 * orc.rng_normal(46, (50,)))
    loss, dl, dvl, kl = om.ppo_loss_fwd_bwd(lg, vl, ac, ol, ad, rt)
    g.update(ppo_logits=lg, ppo_values=vl, ppo_actions=ac, ppo_adv=ad, ppo_ret=rt, ppo_old=ol, ppo_loss=np.array(loss), ppo_dlogits=dl, ppo_dvalues=dvl, ppo_kl=np.array(kl))
    p0 = n(47, (64,)); gr = n(48, (64,), 0.01); p = [p0.copy()]; m = [np.zeros(64)]; vv = [np.zeros(64)]
    for t in range(1, 4): om.adam_step(p, [orc.f32r(gr * t)], m, vv, t, np.float64(np.float32(3e-4)))
    g.update(adam_p0=p0, adam_g=gr, adam_p3=p[0])
    # advantage block: reward normalisation + GAE + advantage normalisation (episode ends inside the buffer)
    rw = orc.f32r(n(50, (300,)) * 3.0 + 1.0); va = n(51, (300,)); tm = (orc.rng_bounded(52, 300, 40) == 0).astype(np.int32)
    adv, ret = orc.gae(rw, va, tm, 0.75, 2.25)
    mean = orc.sum_f64(adv) / adv.size; std = np.sqrt(orc.sum_sq_diff(adv, mean) / adv.size) + 1e-8
    g.update(gae_rewards=rw, gae_values=va, gae_terminals=tm, gae_adv=adv, gae_ret=ret, gae_norm=orc.normalize_slice(adv, mean, std))
    # dueling double-DQN pieces at the crate's batch shape
    dv_, da_ = n(53, (64, 1)), n(54, (64, 5)); dq = n(55, (64, 5))
    qe, qt = n(56, (64, 5)), n(57, (64, 5)); r_ = n(58, (64,)); dn = (orc.rng_bounded(59, 64, 4) == 0).astype(np.float64); ac_ = orc.rng_bounded(60, 64, 5)
    q_ = om.dueling_combine(dv_, da_); bdv, bda = om.dueling_combine_bwd(dq)
    tg = om.dqn_target(qe, qt, r_, dn, np.float64(np.float32(0.99))); ls, ldq = om.dqn_loss_fwd_bwd(q_, ac_, tg)
    g.update(dqn_v=dv_, dqn_a=da_, dqn_q=q_, dqn_dq=dq, dqn_bdv=bdv, dqn_bda=bda, dqn_qe=qe, dqn_qt=qt, dqn_r=r_, dqn_done=dn, dqn_actions=ac_,
             dqn_target=tg, dqn_loss=np.array(ls), dqn_ldq=ldq)
    # batched rollout: 5 simulations x 9 steps of the reference-sized policy, context 3, staggered episode ends
    pol = om.ActorCritic(7)
    st = n(61, (9, 5, 8), 0.5); rs = np.array([[1 if (t * 3 + s_) % 7 == 0 else 0 for s_ in range(5)] for t in range(9)])
    g.update(roll_states=st, roll_resets=rs, roll_probs=om.rollout_reference(pol, st, rs, 3))
    return g


if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(out, **build())
    print(out, os.path.getsize(out), "bytes")
