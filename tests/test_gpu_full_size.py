"""Full-size checks at the benchmark configurations' own sizes, where the f64 oracle would take minutes to hours:
size-independent properties and agreement between independent device implementations (the fp32 CUDA-core kernels
share no code with the tensor-core kernels)."""
import ctypes

import numpy as np
import pytest

import oracle as orc
from oracle import model as om
from gpu_util import TOL, dev, host, normal, rel_err, xavier

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(talos):
    c = talos.torch_context(0)
    yield c
    c.synchronize()


def _gemm(talos, ctx, opA, opB, M, N, K, A, B, mode):
    import torch
    C = torch.empty(M, N, device="cuda:0")
    talos.lib.talos_gemm(ctx.handle, opA, opB, M, N, K, talos.ptr(A), A.shape[1], talos.ptr(B), B.shape[1], talos.ptr(C), N, mode, None)
    return C


def test_gemm_4096_tensor_core_modes_against_the_fp32_kernel_and_linearity(talos, ctx):
    # the north-star GEMM size: 3xTF32 and TF32 against the fp32 FFMA kernel (tolerances of the modes), all three forms
    import torch
    n = 4096
    g = torch.Generator(device="cuda:0"); g.manual_seed(42)
    A = torch.rand(n, n, device="cuda:0", generator=g) * 2 - 1; B = torch.rand(n, n, device="cuda:0", generator=g) * 2 - 1
    for opA, opB in [(0, 0), (0, 1), (1, 0)]:
        ref = _gemm(talos, ctx, opA, opB, n, n, n, A, B, 0).double()
        for mode in (1, 2):
            got = _gemm(talos, ctx, opA, opB, n, n, n, A, B, mode).double()
            err = ((got - ref).norm() / ref.norm()).item()
            assert err <= TOL[mode], (opA, opB, mode, err)
    # linearity in the first operand, fp32-faithful mode: (A1 + A2).B = A1.B + A2.B up to rounding
    A2 = torch.rand(n, n, device="cuda:0", generator=g) * 2 - 1
    lhs = _gemm(talos, ctx, 0, 0, n, n, n, A + A2, B, 1).double()
    rhs = _gemm(talos, ctx, 0, 0, n, n, n, A, B, 1).double() + _gemm(talos, ctx, 0, 0, n, n, n, A2, B, 1).double()
    assert ((lhs - rhs).norm() / rhs.norm()).item() <= 2e-5
    ctx.synchronize()


def test_config5_full_update_modes_agree_and_minibatch_order_is_the_only_coupling(talos, ctx):
    # benchmark configuration 5 at full length: 1 048 576 transitions, minibatch 65 536, 4 epochs = 64 optimizer steps.
    import torch
    N, OBS, HID, ACT, MB = 1048576, 64, 256, 16, 65536
    g = torch.Generator(device="cuda:0"); g.manual_seed(30)
    obs = torch.randn(N, OBS, device="cuda:0", generator=g); act = torch.randint(0, ACT, (N,), device="cuda:0", generator=g, dtype=torch.int32)
    adv = torch.randn(N, device="cuda:0", generator=g); ret = torch.randn(N, device="cuda:0", generator=g)
    rng = np.random.default_rng(34)
    lim = lambda fi, fo: np.sqrt(6.0 / (fi + fo))
    params = dict(w1=rng.uniform(-lim(OBS, HID), lim(OBS, HID), (OBS, HID)), b1=np.zeros(HID), w2=rng.uniform(-lim(HID, HID), lim(HID, HID), (HID, HID)),
                  b2=np.zeros(HID), wp=rng.uniform(-lim(HID, ACT), lim(HID, ACT), (HID, ACT)), bp=np.zeros(ACT),
                  wv=rng.uniform(-lim(HID, 1), lim(HID, 1), (HID, 1)), bv=np.zeros(1))
    results = {}
    old = None
    for mode in (0, 1, 2):
        tr = talos.PPOTrainer(ctx, talos.PpoConfig(OBS, HID, ACT, MB, mode))
        tr.set_params(params)
        if old is None:                                    # the stored rollout log-probabilities: computed once, in fp32 mode
            old = torch.empty(N, device="cuda:0"); tr.log_prob(obs, act, N, old); ctx.synchronize()
        kls = tr.update(obs, act, old, adv, ret, N, 4, 0.0)
        results[mode] = (tr.get_params(), np.array(kls), tr.last_loss())
        tr.close()
    ref, ref_kl, _ = results[0]
    for mode in (1, 2):
        got, kl, loss = results[mode]
        assert np.isfinite(loss) and len(kl) == 4
        errs = {}
        for k in ref:
            init = np.asarray(params[k], dtype=np.float32).reshape(ref[k].shape)
            d_ref = ref[k] - init; d_got = got[k] - init
            errs[k] = (float(np.linalg.norm(got[k] - ref[k]) / (np.linalg.norm(ref[k]) or 1.0)), float(np.linalg.norm(d_got - d_ref) / np.linalg.norm(d_ref)))
        print("mode", mode, {k: "%.1e / %.1e" % v for k, v in errs.items()})
        for k, (w_err, d_err) in errs.items():
            # 64 Adam steps: the normalised update g / (sqrt(v) + eps) is sign-like where gradients are small, so a
            # rounding-level difference in a gradient moves a weight by up to 2 lr per step.  The weights are therefore
            # compared at ten times the single-product tolerance, the learned updates (biases start at zero, so they ARE
            # the update) at an lr-sized bound.
            if k.startswith("w"):
                assert w_err <= 10 * TOL[mode], (mode, k, w_err)
            assert d_err <= (2e-2 if mode == 1 else 5e-2), (mode, k, d_err)
        assert np.allclose(kl, ref_kl, rtol=0.05, atol=1e-6), (mode, kl, ref_kl)
    assert np.all(np.diff(ref_kl) >= -1e-6) or ref_kl[-1] > 0        # the policy does move away from the rollout policy


@pytest.mark.needs_tensor_cores
@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_4096_sampled_rows_against_the_f64_oracle(talos, ctx, mode):
    # the north-star GEMM size against the oracle's f64 restatement of Tensor::matmul (src/autograd.rs:200-258) on 256
    # sampled rows of each result, all three forms; inputs are uniform[-1, 1) fp32 values, identical on both sides
    import torch
    n, rows = 4096, 256
    g = torch.Generator(device="cuda:0"); g.manual_seed(123)
    A = torch.rand(n, n, device="cuda:0", generator=g) * 2 - 1; B = torch.rand(n, n, device="cuda:0", generator=g) * 2 - 1
    Ah, Bh = host(A), host(B)
    pick = np.sort(np.random.default_rng(7).choice(n, rows, replace=False)); pick[0] = 0; pick[-1] = n - 1
    for opA, opB in [(0, 0), (0, 1), (1, 0)]:
        got = host(_gemm(talos, ctx, opA, opB, n, n, n, A, B, mode))[pick]
        lhs = np.ascontiguousarray(Ah[:, pick].T if opA else Ah[pick])        # the sampled rows of op(A)
        rhs = np.ascontiguousarray(Bh.T) if opB else Bh
        ref = orc.matmul(lhs, rhs)
        err = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
        worst = float(np.abs(got - ref).max() / np.abs(ref).max())
        assert err <= TOL[mode] and worst <= 4 * TOL[mode], (opA, opB, mode, err, worst)
    assert ctx.tensor_cores_active


_C5 = {}


def _config5_oracle():
    """Two optimizer steps of benchmark configuration 5 at its own minibatch (65 536 transitions each) through the
    oracle, once per session: stored log-probabilities, the first step's gradient / loss / KL, the parameters after
    both steps and the epoch's mean KL."""
    if _C5:
        return _C5
    OBS, HID, ACT, MB = 64, 256, 16, 65536
    N = 2 * MB
    obs = normal(30, (N, OBS)); act = orc.rng_bounded(31, N, ACT); adv = normal(32, (N,)); ret = normal(33, (N,))
    params = dict(w1=xavier(34, OBS, HID), b1=np.zeros(HID), w2=xavier(35, HID, HID), b2=np.zeros(HID),
                  wp=xavier(36, HID, ACT), bp=np.zeros(ACT), wv=xavier(37, HID, 1), bv=np.zeros(1))
    model = om.MlpActorCritic(params)
    old = orc.f32r(model.log_prob(obs, act))
    g1, loss1, kl1 = model.grads(obs[:MB], act[:MB], old[:MB], adv[:MB], ret[:MB])
    kls, _ = om.ppo_update(model, obs, act, old, adv, ret, 1, MB, lr=np.float64(np.float32(3e-4)))
    _C5.update(obs=obs, act=act, adv=adv, ret=ret, params=params, old=old, g1=g1, loss1=loss1, kl1=kl1, after=model.p, kls=kls, dims=(OBS, HID, ACT, MB, N))
    return _C5


@pytest.mark.needs_tensor_cores
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_config5_full_minibatch_steps_against_the_oracle(talos, ctx, mode):
    # what bench.py times, at the size it times it: minibatch 65 536 (the split-K weight gradients with their 147 slabs,
    # the per-SM column-sum slabs and the gather kernel only take this shape here), against PPO::update's loops
    # (src/ppo.rs:680-769) restated in f64
    c = _config5_oracle()
    OBS, HID, ACT, MB, N = c["dims"]
    tol = TOL[mode]
    d_obs, d_act, d_old, d_adv, d_ret = dev(c["obs"]), dev(c["act"]), dev(c["old"]), dev(c["adv"]), dev(c["ret"])
    tr = talos.PPOTrainer(ctx, talos.PpoConfig(OBS, HID, ACT, MB, mode)); tr.set_params(c["params"])
    import torch
    lp = torch.empty(N, device="cuda:0"); tr.log_prob(d_obs, d_act, N, lp); ctx.synchronize()
    assert rel_err(lp, c["old"]) <= tol
    # step 1: the gradient Adam is about to apply, the mean loss
    tr.step(d_obs, d_act, d_old, d_adv, d_ret, MB)
    got_g = tr.get_grads(); loss = tr.last_loss()
    errs = {k: rel_err(got_g[k], c["g1"][k]) for k in c["g1"]}
    print("mode", mode, "gradient errors", {k: "%.1e" % v for k, v in errs.items()})
    for k, e in errs.items():
        assert e <= 2 * tol, (mode, k, e)              # three chained products per gradient
    assert abs(loss - c["loss1"]) <= max(tol, 2e-6) * abs(c["loss1"]), (loss, c["loss1"])
    # step 2, then the parameters
    tr.step(d_obs[MB:], d_act[MB:], d_old[MB:], d_adv[MB:], d_ret[MB:], MB)
    got = tr.get_params()
    for k in c["after"]:
        init = np.asarray(c["params"][k], dtype=np.float64).reshape(got[k].shape)
        if k.startswith("w"):
            assert rel_err(got[k], c["after"][k]) <= tol, (mode, k, rel_err(got[k], c["after"][k]))
        # the learned update itself (biases start at zero, so they ARE the update): Adam's normalised step is sign-like
        # where a gradient is at rounding level, hence the lr-sized bound
        d_err = rel_err(got[k].astype(np.float64) - init, c["after"][k] - init)
        assert d_err <= (5e-3 if mode != 2 else 5e-2), (mode, k, d_err)
    tr.close()
    # the same two steps through the update loop: per-epoch mean KL, and bit-identical parameters (run-to-run determinism)
    tr2 = talos.PPOTrainer(ctx, talos.PpoConfig(OBS, HID, ACT, MB, mode)); tr2.set_params(c["params"])
    kls = tr2.update(d_obs, d_act, d_old, d_adv, d_ret, N, 1)
    again = tr2.get_params(); tr2.close()
    assert len(kls) == 1 and np.allclose(kls, c["kls"], rtol=1e-3 if mode != 2 else 0.1, atol=1e-7), (kls, c["kls"])
    for k in got:
        assert np.array_equal(got[k], again[k]), k
    if mode:
        assert ctx.tensor_cores_active
