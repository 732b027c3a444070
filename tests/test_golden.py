"""Committed golden vectors (tests/golden/golden.npz, made by tests/golden/make_golden.py): the oracle must keep
reproducing them (CPU), and the CUDA path must match them (GPU)."""
import math
import os

import numpy as np
import pytest

import oracle as orc
from oracle import model as om

G = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz")))


def test_oracle_reproduces_golden_vectors():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec); spec.loader.exec_module(mg)
    fresh = mg.build()
    assert set(fresh) == set(G)
    for k in G:
        assert np.allclose(fresh[k], G[k], rtol=1e-12, atol=1e-14), k
    # and the crate's constants are what the oracle computes
    assert np.array_equal(orc.matmul(G["kat_matmul_A"], G["kat_matmul_x"]).ravel(), G["kat_matmul_y"])
    dA, dx = orc.matmul_bwd(G["kat_matmul_A"], G["kat_matmul_x"], np.ones((2, 1)))
    assert np.allclose(dx.ravel(), G["kat_matmul_dx"]) and np.allclose(dA.ravel(), G["kat_matmul_dA"])
    assert np.array_equal(orc.transpose(G["kat_transpose_in"], 0, 1).ravel(), G["kat_transpose_out"])


@pytest.mark.gpu
def test_cuda_path_matches_golden_vectors(talos):
    import ctypes as C
    import torch
    from gpu_util import dev, host, rel_err
    ctx = talos.torch_context(0)
    L, P = talos.lib, talos.ptr
    e = lambda n, m=1: torch.empty(n, m, device="cuda:0") if m > 1 else torch.empty(n, device="cuda:0")
    for mode in (0, 1):
        A, B, Gd = dev(G["mm_A"]), dev(G["mm_B"]), dev(G["mm_G"])
        Cm = e(17, 9); dA = e(17, 13); dB = e(13, 9)
        L.talos_gemm(ctx.handle, 0, 0, 17, 9, 13, P(A), 13, P(B), 9, P(Cm), 9, mode, None)
        L.talos_gemm(ctx.handle, 0, 1, 17, 13, 9, P(Gd), 9, P(B), 9, P(dA), 13, mode, None)
        L.talos_gemm(ctx.handle, 1, 0, 13, 9, 17, P(A), 13, P(Gd), 9, P(dB), 9, mode, None)
        ctx.synchronize()
        assert rel_err(Cm, G["mm_C"]) <= 1e-5 and rel_err(dA, G["mm_dA"]) <= 1e-5 and rel_err(dB, G["mm_dB"]) <= 1e-5
        # MLP through talos_linear_fwd / bwd
        h = [dev(G["mlp_X"])]; dims = [8, 16, 16, 5]; acts = [2, 2, 0]
        W = [dev(G["mlp_W%d" % i]) for i in range(3)]; b = [dev(G["mlp_b%d" % i]) for i in range(3)]
        for i in range(3):
            y = e(33, dims[i + 1]); L.talos_linear_fwd(ctx.handle, P(h[-1]), P(W[i]), P(b[i]), P(y), None, 33, dims[i], dims[i + 1], acts[i], mode); h.append(y)
        g = dev(G["mlp_dY"])
        for i in (2, 1, 0):
            dx = e(33, dims[i]); dW = torch.empty_like(W[i]); db = torch.empty_like(b[i])
            L.talos_linear_bwd(ctx.handle, P(h[i]), P(W[i]), P(h[i + 1]), P(g), P(dx), P(dW), P(db), 33, dims[i], dims[i + 1], acts[i], mode, 0)
            ctx.synchronize()
            assert rel_err(dW, G["mlp_dW%d" % i]) <= 1e-5 and rel_err(db, G["mlp_db%d" % i]) <= 1e-5, i
            g = dx
        assert rel_err(h[3], G["mlp_Y"]) <= 1e-5 and rel_err(g, G["mlp_dX"]) <= 1e-5
    # RMSNorm
    x, gam, gy = dev(G["rms_x"]), dev(G["rms_gamma"]), dev(G["rms_gy"]); y = e(19, 24); inv = e(19); dx = e(19, 24); dg = e(24)
    L.talos_rmsnorm_fwd(ctx.handle, P(x), P(gam), 1e-5, 19, 24, P(y), P(inv))
    L.talos_rmsnorm_bwd(ctx.handle, P(gy), P(x), P(gam), P(inv), 19, 24, P(dx), P(dg), 0)
    ctx.synchronize()
    assert rel_err(y, G["rms_y"]) <= 1e-6 and rel_err(dx, G["rms_dx"]) <= 1e-5 and rel_err(dg, G["rms_dgamma"]) <= 1e-5
    # RoPE
    c = e(64); s = e(64); L.talos_rope_table(ctx.handle, 8, 16, 10000.0, P(c), P(s))
    xr = dev(G["rope_x"]); yr = torch.empty_like(xr)
    L.talos_rope(ctx.handle, P(xr), P(yr), P(c), P(s), 64, 2, 5, 3, 8, 2, 0, 0); ctx.synchronize(); assert rel_err(yr, G["rope_token"]) <= 1e-6
    L.talos_rope(ctx.handle, P(xr), P(yr), P(c), P(s), 64, 10, 3, 1, 8, 0, 0, 0); ctx.synchronize(); assert rel_err(yr, G["rope_head"]) <= 1e-6
    L.talos_rope(ctx.handle, P(xr), P(yr), P(c), P(s), 64, 10, 3, 1, 8, 0, 1, 0); ctx.synchronize(); assert rel_err(yr, G["rope_head_bwd"]) <= 1e-6
    # softmax / attention
    sx, sg = dev(G["sm_x"]), dev(G["sm_g"]); sy = e(11, 20); sdx = e(11, 20)
    sy_ref = dev(G["sm_y"])
    L.talos_softmax_fwd(ctx.handle, P(sx), P(sy), 11, 20, 1.0, 0); L.talos_softmax_bwd(ctx.handle, P(sy_ref), P(sg), P(sdx), 11, 20, 1.0, 0)
    ctx.synchronize(); assert rel_err(sy, G["sm_y"]) <= 2e-6 and rel_err(sdx, G["sm_dx"]) <= 1e-5
    q, k, v, go = dev(G["att_q"]), dev(G["att_k"]), dev(G["att_v"]), dev(G["att_go"]); O = torch.empty_like(v); Pr = torch.empty(3, 10, 10, device="cuda:0")
    dq = torch.empty_like(q); dk = torch.empty_like(k); dv = torch.empty_like(v); sc = 1.0 / math.sqrt(12.0)
    L.talos_attention_fwd(ctx.handle, P(q), P(k), P(v), P(O), P(Pr), 3, 10, 12, 6, sc, 0, 0)
    L.talos_attention_bwd(ctx.handle, P(q), P(k), P(v), P(Pr), P(go), P(dq), P(dk), P(dv), 3, 10, 12, 6, sc, 0)
    ctx.synchronize()
    for a, name in ((O, "att_O"), (Pr, "att_P"), (dq, "att_dq"), (dk, "att_dk"), (dv, "att_dv")):
        assert rel_err(a, G[name]) <= 2e-5, name
    # PPO loss and Adam
    n, A = 50, 5
    dl = e(n, A); dvv = e(n); st = torch.zeros(4, device="cuda:0")
    t_ = {k: dev(G["ppo_" + k]) for k in ("logits", "values", "actions", "old", "adv", "ret")}      # keep every input alive for the call
    L.talos_ppo_loss_fwd_bwd(ctx.handle, P(t_["logits"]), A, P(t_["values"]), 1, P(t_["actions"]), P(t_["old"]), P(t_["adv"]),
                             P(t_["ret"]), n, A, 0.2, 0.5, 0.01, float(n), P(dl), A, P(dvv), 1, P(st))
    ctx.synchronize()
    assert rel_err(dl, G["ppo_dlogits"]) <= 1e-5 and rel_err(dvv, G["ppo_dvalues"]) <= 1e-5
    assert abs(host(st)[0] / n - float(G["ppo_loss"])) <= 1e-5 and abs(host(st)[1] - float(G["ppo_kl"])) <= 1e-4
    p = dev(G["adam_p0"]); m = torch.zeros(64, device="cuda:0"); vv = torch.zeros(64, device="cuda:0")
    for t in range(1, 4):
        gt = dev(orc.f32r(G["adam_g"] * t))
        L.talos_adam_step(ctx.handle, P(p), P(gt), P(m), P(vv), 64, t, 3e-4, 0.9, 0.999, 1e-8, 1.0, 0.0)
    ctx.synchronize(); assert rel_err(p, G["adam_p3"]) <= 1e-6
    # advantage block
    n = 300; rw, va = dev(G["gae_rewards"]), dev(G["gae_values"]); tm = torch.from_numpy(G["gae_terminals"].astype(np.int32)).cuda()
    adv = e(n); ret = e(n); nrm = e(n)
    L.talos_gae(ctx.handle, P(rw), P(va), P(tm), n, 0.99, 0.95, 0.75, 2.25, P(adv), P(ret))
    L.talos_normalize_slice(ctx.handle, P(adv), n, P(nrm), None)
    ctx.synchronize()
    assert rel_err(adv, G["gae_adv"]) <= 1e-5 and rel_err(ret, G["gae_ret"]) <= 1e-5 and rel_err(nrm, G["gae_norm"]) <= 1e-5
    # dueling double-DQN pieces
    B, A = 64, 5
    v_, a_, dq_ = dev(G["dqn_v"]), dev(G["dqn_a"]), dev(G["dqn_dq"]); q_ = e(B, A); bdv = e(B, 1); bda = e(B, A)
    L.talos_dueling_combine_fwd(ctx.handle, P(v_), P(a_), P(q_), B, A)
    L.talos_dueling_combine_bwd(ctx.handle, P(dq_), P(bdv), P(bda), B, A, 0)
    qe, qt, r_, dn = dev(G["dqn_qe"]), dev(G["dqn_qt"]), dev(G["dqn_r"]), dev(G["dqn_done"]); tg = e(B)
    L.talos_dqn_target(ctx.handle, P(qe), P(qt), P(r_), P(dn), 0.99, P(tg), B, A)
    acts = torch.from_numpy(G["dqn_actions"].astype(np.int32)).cuda(); ls = e(1); ldq = e(B, A)
    L.talos_dqn_loss_fwd_bwd(ctx.handle, P(q_), P(acts), P(tg), P(ls), P(ldq), B, A)
    ctx.synchronize()
    assert rel_err(q_, G["dqn_q"]) <= 1e-6 and rel_err(bdv, G["dqn_bdv"]) <= 1e-6 and rel_err(bda, G["dqn_bda"]) <= 1e-6
    assert rel_err(tg, G["dqn_target"]) <= 1e-6 and abs(host(ls)[0] - float(G["dqn_loss"])) <= 1e-5 * float(G["dqn_loss"]) and rel_err(ldq, G["dqn_ldq"]) <= 1e-5
    ctx.close()
