"""Full-size checks at the benchmark configurations' own sizes, where the f64 oracle would take minutes to hours:
size-independent properties and agreement between independent device implementations (the fp32 CUDA-core kernels
share no code with the tensor-core kernels)."""
import ctypes

import numpy as np
import pytest

from gpu_util import TOL

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
