"""Error paths on the device, exercised without faulting, trapping or hanging anything:

* the device-side error word must surface from EVERY entry point that blocks on the stream (not only from
  talos_ctx_synchronize), as TALOS_ERR_TIMEOUT or TALOS_ERR_ARG, and be cleared by the report;
* an action index outside [0, n_actions) in device memory is skipped and reported, never dereferenced;
* a bounded wait inside the tensor-core GEMM that runs out (a k-block the loader leaves out on purpose, a short
  poll limit) makes the kernel give up cleanly: status TIMEOUT, context still usable, next product correct;
* the slice primitives of src/simd.rs and the softmax argument check.
"""
import ctypes
import math

import numpy as np
import pytest

import oracle as orc
from gpu_util import TOL, dev, host, normal, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(talos):
    c = talos.torch_context(0)
    yield c
    c.synchronize()


def _expect(talos, status, fn):
    with pytest.raises(talos.TalosError) as e:
        fn()
    assert e.value.status == status, (e.value.status, str(e.value))


def test_device_error_word_surfaces_from_every_blocking_entry_point(talos, ctx):
    import torch
    x = torch.arange(8, dtype=torch.float32, device="cuda:0")
    h32 = np.empty(8, np.float32); h64 = np.empty(8, np.float64)
    tr = talos.PPOTrainer(ctx, talos.PpoConfig(8, 32, 5, 64, 0))
    n = tr.n_params
    flat = np.zeros(n, np.float32); tr.set_params(flat)
    obs = torch.randn(64, 8, device="cuda:0"); act = torch.zeros(64, dtype=torch.int32, device="cuda:0")
    old = torch.zeros(64, device="cuda:0"); adv = torch.randn(64, device="cuda:0"); ret = torch.randn(64, device="cuda:0")
    tr.step(obs, act, old, adv, ret, 64)
    blocking = {
        "synchronize": lambda: ctx.synchronize(),
        "copy_to_host": lambda: talos.lib.talos_copy_to_host(ctx.handle, talos.ptr(h32), talos.ptr(x), 32),
        "download_f64": lambda: talos.lib.talos_download_f64(ctx.handle, talos.ptr(h64), talos.ptr(x), 8),
        "get_params": lambda: tr.get_params(),
        "last_loss": lambda: tr.last_loss(),
        "update": lambda: tr.update(obs, act, old, adv, ret, 64, 2),
        "update_host": lambda: tr.update(obs.cpu().numpy(), act.cpu().numpy(), old.cpu().numpy(), adv.cpu().numpy(), ret.cpu().numpy(), 64, 2, host=True),
    }
    for name, call in blocking.items():
        for code, status in ((1007, talos.ERR_TIMEOUT), (2003, talos.ERR_TIMEOUT), (3000, talos.ERR_ARG)):
            talos.lib.talos_debug_set_device_status(ctx.handle, code)
            _expect(talos, status, call)
            call()                                     # the report cleared the word: the same call now succeeds
    assert np.array_equal(h32, np.arange(8, dtype=np.float32)) and np.array_equal(h64, np.arange(8.0))
    tr.close()


def test_out_of_range_actions_are_skipped_and_reported(talos, ctx):
    import torch
    A = 5
    # PPO: stored log-probabilities and the loss kernel
    tr = talos.PPOTrainer(ctx, talos.PpoConfig(8, 32, A, 128, 0))
    rng = np.random.default_rng(3)
    tr.set_params(rng.standard_normal(tr.n_params).astype(np.float32) * 0.1)
    obs = torch.randn(128, 8, device="cuda:0"); act = torch.randint(0, A, (128,), dtype=torch.int32, device="cuda:0")
    bad = act.clone(); bad[17] = A; bad[90] = -1
    out = torch.empty(128, device="cuda:0")
    tr.log_prob(obs, act, 128, out); ctx.synchronize()
    good = out.clone()
    tr.log_prob(obs, bad, 128, out)
    _expect(talos, talos.ERR_ARG, ctx.synchronize)
    keep = torch.ones(128, dtype=torch.bool, device="cuda:0"); keep[17] = False; keep[90] = False
    assert torch.equal(out[keep], good[keep]) and float(out[17]) == 0.0 and float(out[90]) == 0.0
    adv = torch.randn(128, device="cuda:0"); ret = torch.randn(128, device="cuda:0")
    tr.step(obs, bad, good, adv, ret, 128)
    _expect(talos, talos.ERR_ARG, tr.last_loss)
    tr.step(obs, act, good, adv, ret, 128); assert np.isfinite(tr.last_loss())
    tr.close()
    # DQN loss: the sample is left out of the loss and gets a zero gradient row
    B = 64
    q = torch.randn(B, A, device="cuda:0"); tgt = torch.randn(B, device="cuda:0")
    a = torch.randint(0, A, (B,), dtype=torch.int32, device="cuda:0"); a_bad = a.clone(); a_bad[5] = 1 << 20
    loss = torch.zeros(1, device="cuda:0"); dq = torch.full((B, A), 7.0, device="cuda:0")
    talos.lib.talos_dqn_loss_fwd_bwd(ctx.handle, talos.ptr(q), talos.ptr(a_bad), talos.ptr(tgt), talos.ptr(loss), talos.ptr(dq), B, A)
    _expect(talos, talos.ERR_ARG, ctx.synchronize)
    assert float(dq[5].abs().sum()) == 0.0
    qs = q[torch.arange(B, device="cuda:0"), a.long()]; d = (qs - tgt).double(); d[5] = 0
    assert abs(float(loss) - float((d * d).sum() / B)) <= 1e-5 * max(1.0, float(loss))
    talos.lib.talos_dqn_loss_fwd_bwd(ctx.handle, talos.ptr(q), talos.ptr(a), talos.ptr(tgt), talos.ptr(loss), talos.ptr(dq), B, A)
    ctx.synchronize()


@pytest.mark.parametrize("mode", [2, 1])
def test_bounded_wait_in_the_gemm_gives_up_cleanly(talos, ctx, mode):
    import torch
    M, N, K = 1024, 256, 256
    g = torch.Generator(device="cuda:0"); g.manual_seed(11)
    A = torch.rand(M, K, device="cuda:0", generator=g) - 0.5; B = torch.rand(K, N, device="cuda:0", generator=g) - 0.5
    C = torch.empty(M, N, device="cuda:0")
    call = lambda m: talos.lib.talos_gemm(ctx.handle, 0, 0, M, N, K, talos.ptr(A), K, talos.ptr(B), N, talos.ptr(C), N, m, None)
    call(mode); ctx.synchronize()                      # first use runs the start-up self-check
    assert ctx.tensor_cores_active
    ref = (A.double() @ B.double())
    assert float((C.double() - ref).norm() / ref.norm()) <= TOL[mode]
    try:
        talos.lib.talos_debug_gemm_stall(ctx.handle, 1, 20000)       # the second k-block of CTA 0's first tile never arrives
        call(mode)
        _expect(talos, talos.ERR_TIMEOUT, ctx.synchronize)           # the kernel returned by itself; the word was raised
    finally:
        talos.lib.talos_debug_gemm_stall(ctx.handle, -1, 0)
    C.zero_(); call(mode); ctx.synchronize()                         # same context, same kernel: correct again
    assert float((C.double() - ref).norm() / ref.norm()) <= TOL[mode]
    assert ctx.tensor_cores_active


def test_simd_slice_primitives(talos, ctx):
    import torch
    # the reference's own known-answer tests (src/dbn.rs:391-415) ...
    row = np.array([1.0, 2.5, -3.0, 4.0, -5.5, 6.25, 7.75, -8.0]); out = torch.zeros(8, device="cuda:0")
    d_row = dev(row)
    talos.lib.talos_axpy(ctx.handle, talos.ptr(out), talos.ptr(d_row), 0.75, 8); ctx.synchronize()
    assert np.abs(host(out) - 0.75 * row).max() < 1e-9 * 8                 # values are exact in fp32
    a = np.array([1.5, -2.0, 3.25, 4.0, -5.0, 6.5, -7.25, 8.0]); b = np.array([0.5, 1.25, -2.0, 3.0, 4.5, -5.5, 6.0, -7.0])
    d = torch.zeros(1, device="cuda:0"); d_a, d_b = dev(a), dev(b)      # (named: a temporary would be freed, and its memory reused, before the call)
    talos.lib.talos_dot(ctx.handle, talos.ptr(d_a), talos.ptr(d_b), 8, talos.ptr(d), 0); ctx.synchronize()
    assert abs(float(d) - float(np.dot(a, b))) < 1e-9 * 200                # -154.0, exact in fp32
    # ... and against the oracle's restatement at lengths around the vector width, unaligned starts, large n
    for n, off in [(1, 0), (3, 1), (4, 0), (1000, 0), (1001, 3), (1 << 20, 0), ((1 << 20) + 5, 1)]:
        X = normal(n, (n + off,)); Y = normal(n + 1, (n + off,)); Z = normal(n + 2, (n + off,))
        x, y, z = dev(X), dev(Y), dev(Z)
        talos.lib.talos_axpy(ctx.handle, talos.ptr(z) + 4 * off, talos.ptr(x) + 4 * off, -1.25, n); ctx.synchronize()
        assert rel_err(z[off:], orc.add_scaled_row(Z[off:].copy(), X[off:], -1.25)) <= 1e-6
        z = dev(Z)
        talos.lib.talos_vector_fma(ctx.handle, talos.ptr(z) + 4 * off, talos.ptr(x) + 4 * off, talos.ptr(y) + 4 * off, n); ctx.synchronize()
        assert rel_err(z[off:], orc.vector_fma(Z[off:].copy(), X[off:], Y[off:])) <= 1e-6
        talos.lib.talos_dot(ctx.handle, talos.ptr(x) + 4 * off, talos.ptr(y) + 4 * off, n, talos.ptr(d), 0); ctx.synchronize()
        ref = orc.dot_product(X[off:], Y[off:])
        assert abs(float(d) - ref) <= 1e-5 * max(1.0, float(np.sqrt(n))), (n, float(d), ref)
        z = dev(Z)
        talos.lib.talos_vector_scale(ctx.handle, talos.ptr(z) + 4 * off, 0.3, n); ctx.synchronize()
        assert rel_err(z[off:], Z[off:] * np.float64(np.float32(0.3))) <= 1e-6
        z = dev(Z); s = torch.zeros(1, device="cuda:0")
        talos.lib.talos_softmax_exp_sum(ctx.handle, talos.ptr(z) + 4 * off, n, talos.ptr(s)); ctx.synchronize()
        e = np.exp(Z[off:] - Z[off:].max())
        assert rel_err(z[off:], e) <= 2e-6 and abs(float(s) - e.sum()) <= 1e-5 * e.sum()
    talos.lib.talos_softmax_exp_sum(ctx.handle, None, 0, talos.ptr(s)); ctx.synchronize(); assert float(s) == 0.0   # empty row (src/simd.rs:336-338)


def test_softmax_rejects_a_causal_period_longer_than_the_row(talos, ctx):
    import torch
    x = torch.zeros(4, 100, device="cuda:0"); y = torch.empty_like(x)
    _expect(talos, talos.ERR_SHAPE, lambda: talos.lib.talos_softmax_fwd(ctx.handle, talos.ptr(x), talos.ptr(y), 4, 100, 1.0, 101))
    _expect(talos, talos.ERR_SHAPE, lambda: talos.lib.talos_softmax_fwd(ctx.handle, talos.ptr(x), talos.ptr(y), 4, 100, 1.0, -1))
    # an odd row length with the longest legal period: row r sees columns 0..r
    rows = n = 100
    X = normal(9, (rows, n), 2.0); scale = 1.0 / math.sqrt(7.0)
    y = torch.empty(rows, n, device="cuda:0")
    d_x = dev(X)
    talos.lib.talos_softmax_fwd(ctx.handle, talos.ptr(d_x), talos.ptr(y), rows, n, scale, n); ctx.synchronize()
    assert rel_err(y, orc.softmax(orc.f32r(X) * np.float64(np.float32(scale)), n)) <= 2e-6


def test_caching_allocator_reuses_blocks_and_refuses_foreign_pointers(talos, ctx):
    stats = (ctypes.c_int64 * 4)()
    def st():
        talos.lib.talos_ctx_memory_stats(ctx.handle, stats); return list(stats)
    talos.lib.talos_ctx_trim(ctx.handle)
    base = st()
    ptrs = []
    for _ in range(3):
        for nbytes in (100, 4096, 5000, 3 << 20):
            p = ctypes.c_void_p(); talos.lib.talos_malloc(ctx.handle, nbytes, ctypes.byref(p)); ptrs.append(p)
        for p in ptrs:
            talos.lib.talos_free(ctx.handle, p)
        ptrs = []
    after = st()
    assert after[2] - base[2] == 4 and after[3] - base[3] == 8      # four driver allocations, then everything from the cache
    assert after[0] == base[0] and after[1] - base[1] == 256 + 4096 + 8192 + (3 << 20)
    _expect(talos, talos.ERR_ARG, lambda: talos.lib.talos_free(ctx.handle, ctypes.c_void_p(0x1000)))
    talos.lib.talos_ctx_trim(ctx.handle)
    assert st()[1] == 0


def test_launch_timeline_reports_every_launch_in_order(talos, ctx):
    # measurement aid: one event behind every launch between begin and end; times are positive, names in launch order
    import torch
    a = torch.randn(4096, 256, device="cuda:0"); out = torch.empty(256, device="cuda:0")
    l0 = ctx.launches
    ctx.timeline_begin()
    for _ in range(3):
        talos.lib.talos_colsum(ctx.handle, talos.ptr(a), talos.ptr(out), 4096, 256, 0)
    marks = ctx.timeline_end()
    assert len(marks) == ctx.launches - l0 and len(marks) >= 3
    assert all(us > 0 for _, us in marks) and all(name.startswith("colsum") for name, _ in marks)
    l1 = ctx.launches
    talos.lib.talos_colsum(ctx.handle, talos.ptr(a), talos.ptr(out), 4096, 256, 0)        # recording is off again
    ctx.synchronize()
    assert ctx.launches > l1
    assert torch.allclose(out, a.sum(0), rtol=1e-4, atol=1e-3)
