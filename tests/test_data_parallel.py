"""Data-parallel PPO update: G ranks x n samples must equal one rank x G*n samples.

CPU part (gloo, world_size 2): the exchange protocol itself -- local gradient SUMS plus a {loss, kl, count} tail,
one all-reduce per optimizer step, division by the global count, identical Adam on every rank -- driven with the
oracle's gradients.  GPU part (needs >= 2 devices): the library's trainer with its NCCL exchange."""
import os
import socket
import subprocess
import sys
import tempfile

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return str(p)


def launch(kind, world, env=None, timeout=240):
    """Runs `world` worker processes and returns their results.  The group is torn down as soon as one rank fails or
    the time runs out: a rank that exits early would otherwise leave its peers waiting inside a collective, holding
    their GPUs."""
    import time
    port = free_port(); outs = []; procs = []; logs = []
    d = tempfile.mkdtemp()
    try:
        for r in range(world):
            out = os.path.join(d, "r%d.npz" % r); outs.append(out)
            log = open(os.path.join(d, "r%d.log" % r), "w+"); logs.append(log)
            procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dp_worker.py"), kind, str(r), str(world), port, out],
                                          stdout=log, stderr=subprocess.STDOUT, env=dict(os.environ, **(env or {}))))
        deadline = time.time() + timeout
        failed = None
        while failed is None and any(p.poll() is None for p in procs):
            if time.time() > deadline:
                failed = "timed out after %d s" % timeout
            for r, p in enumerate(procs):
                if p.poll() not in (None, 0):
                    failed = "rank %d exited with %d" % (r, p.returncode)
            time.sleep(0.05)
        for r, p in enumerate(procs):
            if failed is None and p.returncode != 0:
                failed = "rank %d exited with %d" % (r, p.returncode)

        def text(f):
            f.flush(); f.seek(0); return f.read()
        assert failed is None, failed + "\n" + "\n".join(text(f)[-4000:] for f in logs)
        return [dict(np.load(o)) for o in outs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        for p in procs:
            p.wait()
        for f in logs:
            f.close()


def single_rank_reference():
    sys.path.insert(0, HERE)
    import dp_worker as w
    import oracle as orc
    from oracle import model as om
    obs, act, adv, ret, params = w.problem()
    model = om.MlpActorCritic(params)
    old = orc.f32r(model.log_prob(obs, act))
    kls, _ = om.ppo_update(model, obs, act, old, adv, ret, w.EPOCHS, w.MB, lr=np.float64(np.float32(3e-4)))
    return model.p, kls


def test_two_gloo_ranks_equal_one_rank_on_the_global_batch():
    ref, ref_kls = single_rank_reference()
    res = launch("cpu", 2)
    for k in ref:
        assert np.array_equal(res[0][k], res[1][k]), "ranks diverged: " + k        # identical Adam on identical reduced gradients
        assert np.allclose(res[0][k], ref[k], rtol=1e-9, atol=1e-12), k
    assert np.allclose(res[0]["kls"], ref_kls, rtol=1e-9)


@pytest.mark.gpu
@pytest.mark.parametrize("mode,path", [(0, "peer"), (1, "peer"), (1, "nccl")])
def test_two_gpu_ranks_equal_one_gpu_rank_and_the_oracle(mode, path):
    # both gradient exchanges: the fused peer-memory kernel (sum in rank order + Adam + weight preparation) and the NCCL
    # all-reduce it replaces
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ref, ref_kls = single_rank_reference()
    env = {"TALOS_TEST_MODE": str(mode), "NCCL_NVLS_ENABLE": "0"}
    if path == "nccl":
        env["TALOS_COMM_NO_P2P"] = "1"
    two = launch("gpu", 2, env); one = launch("gpu", 1, env)
    assert bool(two[0]["peer"]) == (path == "peer") and bool(two[1]["peer"]) == (path == "peer")
    for k in ref:
        assert np.array_equal(two[0][k], two[1][k]), "ranks diverged: " + k
        d = np.linalg.norm(ref[k]); d = d if d > 0 else 1.0
        assert np.linalg.norm(two[0][k] - one[0][k].reshape(two[0][k].shape)) <= 1e-5 * max(np.linalg.norm(one[0][k]), 1e-3), k
        if k.startswith("w"):
            assert np.linalg.norm(two[0][k] - ref[k].reshape(two[0][k].shape)) <= 1e-5 * d, k
    assert np.allclose(two[0]["kls"], ref_kls, rtol=1e-3, atol=1e-8)


@pytest.mark.gpu
def test_a_rank_that_never_publishes_makes_the_others_give_up_cleanly():
    # failure detection without a fault: the last rank skips one publication (a host-side switch); the other rank's
    # bounded wait runs out, its kernel returns, the error word surfaces as TALOS_ERR_TIMEOUT and its weights are untouched
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = launch("gpu_stall", 2, {"TALOS_TEST_MODE": "1", "NCCL_NVLS_ENABLE": "0"})
    assert bool(res[0]["peer"]) and int(res[0]["status"]) == 6 and bool(res[0]["unchanged"])      # rank 0 gave up: TALOS_ERR_TIMEOUT
    assert int(res[1]["status"]) == 0 and not bool(res[1]["unchanged"])                           # rank 1 saw rank 0's publication and stepped
