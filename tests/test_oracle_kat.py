"""Pins the CPU oracle against every known-answer test the reference crate holds for this path.
Each test names the reference test it replays."""
import math

import numpy as np

import oracle as orc
from oracle import model as om


def test_add_scaled_row_matches_scalar():
    # src/dbn.rs:391-403
    row = np.array([1.0, 2.5, -3.0, 4.0, -5.5, 6.25, 7.75, -8.0])
    got = orc.add_scaled_row(np.zeros(8), row, 0.75)
    assert np.all(np.abs(got - 0.75 * row) < 1e-9)


def test_dot_product_matches_scalar():
    # src/dbn.rs:406-415
    a = [1.5, -2.0, 3.25, 4.0, -5.0, 6.5, -7.25, 8.0]
    b = [0.5, 1.25, -2.0, 3.0, 4.5, -5.5, 6.0, -7.0]
    exp = 0.0
    for x, y in zip(a, b):
        exp += x * y
    assert abs(orc.dot_product(a, b) - exp) < 1e-9


def test_primitives_odd_lengths():
    rng = np.random.default_rng(0)
    for n in (0, 1, 3, 4, 7, 8, 9, 17, 64, 129):
        a = rng.standard_normal(n); b = rng.standard_normal(n); d = rng.standard_normal(n)
        assert np.allclose(orc.add_scaled_row(d, a, -1.25), d - 1.25 * a, atol=1e-12)
        assert abs(orc.dot_product(a, b) - float(a @ b)) < 1e-10
        assert np.allclose(orc.vector_fma(d, a, b), d + a * b, atol=1e-12)
        assert np.allclose(orc.vector_scale(a, 3.0), 3.0 * a)
        e, s = orc.softmax_exp_sum(a)
        if n == 0:
            assert s == 0.0                                           # src/simd.rs:335-337
        else:
            assert np.allclose(e, np.exp(a - a.max())) and abs(s - e.sum()) < 1e-12


def test_sum_f64_matches_scalar():
    # src/ppo.rs:1051-1059
    v = [1.0, -2.5, 3.25, 4.0, -5.0, 6.5, 7.75, -8.0, 9.0]
    assert abs(orc.sum_f64(v) - sum(v)) < 1e-9


def test_normalize_slice_zero_mean_unit_std():
    # src/ppo.rs:1062-1071
    v = np.arange(1.0, 10.0)
    mean = orc.sum_f64(v) / v.size
    std = math.sqrt(orc.sum_sq_diff(v, mean) / v.size) + 1e-8
    norm = orc.normalize_slice(v, mean, std)
    assert abs(orc.sum_f64(norm) / norm.size) < 1e-9
    assert abs(math.sqrt(orc.sum_sq_diff(norm, 0.0) / norm.size) - 1.0) < 1e-6


def test_grad_check_matmul():
    # src/grad_check.rs:30-63: A=[[2,3],[4,5]], x=[1,2]^T, L=sum(Ax) -> dx=[6,8], dA=[1,2,1,2]
    A = np.array([[2.0, 3.0], [4.0, 5.0]]); x = np.array([[1.0], [2.0]])
    y = orc.matmul(A, x)
    assert np.array_equal(y.ravel(), [8.0, 14.0])
    dA, dx = orc.matmul_bwd(A, x, np.ones((2, 1)))
    assert np.all(np.abs(dx.ravel() - [6.0, 8.0]) < 1e-6)
    assert np.all(np.abs(dA.ravel() - [1.0, 2.0, 1.0, 2.0]) < 1e-6)


def test_matmul_1d_lhs_and_serial_threshold():
    # src/autograd.rs:203-207 (1-D lhs), :222 (serial below 32768 MACs): both paths agree with numpy
    rng = np.random.default_rng(1)
    for (M, K, N) in [(1, 8, 5), (3, 17, 9), (31, 32, 33), (64, 64, 64), (130, 70, 50)]:
        A = rng.standard_normal((M, K)); B = rng.standard_normal((K, N)); G = rng.standard_normal((M, N))
        assert np.allclose(orc.matmul(A, B), A @ B, atol=1e-11)
        dA, dB = orc.matmul_bwd(A, B, G)
        assert np.allclose(dA, G @ B.T, atol=1e-11) and np.allclose(dB, A.T @ G, atol=1e-11)
    v = rng.standard_normal(8); B = rng.standard_normal((8, 5))
    assert orc.matmul(v, B).shape == (5,)


def test_matmul_backward_accumulates():
    # src/autograd.rs:304, :346: gradients are += into the parents
    rng = np.random.default_rng(2)
    A = rng.standard_normal((4, 3)); B = rng.standard_normal((3, 5)); G = rng.standard_normal((4, 5))
    dA0 = np.ones((4, 3)); dB0 = np.full((3, 5), 2.0)
    dA, dB = orc.matmul_bwd(A, B, G, dA0.copy(), dB0.copy())
    assert np.allclose(dA, 1.0 + G @ B.T) and np.allclose(dB, 2.0 + A.T @ G)


def test_grad_check_broadcast():
    # src/grad_check.rs:66-90: z = x + broadcast(y); dL/dx=[1,1], dL/dy=2  (bias path of Linear)
    z = orc.bias_add(np.array([[1.0], [2.0]]), np.array([10.0]))
    assert np.array_equal(z.ravel(), [11.0, 12.0])
    assert orc.bias_bwd(np.ones((2, 1)), 1)[0] == 2.0


def test_tensor_transpose():
    # src/transformer.rs:1212-1225
    t = orc.transpose(np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]), 0, 1)
    assert t.shape == (3, 2) and np.array_equal(t.ravel(), [1, 4, 2, 5, 3, 6])
    x = np.random.default_rng(3).standard_normal((2, 3, 4, 5))
    assert np.array_equal(orc.transpose(x, 1, 2), x.swapaxes(1, 2))
    g = np.random.default_rng(4).standard_normal((2, 4, 3, 5))
    assert np.array_equal(orc.transpose(g, 1, 2, backward=True), g.swapaxes(1, 2))


def test_lcg_rand_half_range():
    # src/autograd.rs:114-124: r = (x>>33)/u32::MAX lies in [0, 0.5): rand(-1,1) is all negative
    a = orc.lcg_rand((1024,), -1.0, 1.0, 42)
    assert a.min() >= -1.0 and a.max() < 0.0
    x = (42 * 6364136223846793005 + 1) % (1 << 64)
    assert a[0] == -1.0 + ((x >> 33) / 4294967295.0) * 2.0
    W, b = om.linear_init_lcg(8, 64, True, 7)
    assert W.max() < 0.0 and np.all(b == 0.0) and W.min() >= -math.sqrt(6.0 / 72)


def test_xoshiro_reference_vectors():
    # src/rng.rs:14-70.  Known answers of the published generators: SplitMix64 seeded with 0 yields
    # 0xe220a8397b1dcdaf first; xoshiro256** from state {1,2,3,4} yields 11520 first.
    u = orc.rng_u64(0, 4)
    s = [0xe220a8397b1dcdaf, 0x6e789e6aa1b965f4, 0x06c45d188009454f, 0xf88bb8a8724c81ec]   # SplitMix64(0) stream
    rotl = lambda x, k: ((x << k) | (x >> (64 - k))) & (2**64 - 1)
    exp = []
    for _ in range(4):
        exp.append((rotl((s[1] * 5) & (2**64 - 1), 7) * 9) & (2**64 - 1))
        t = (s[1] << 17) & (2**64 - 1)
        s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl(s[3], 45)
    assert [int(v) for v in u] == exp
    f = orc.rng_uniform(5, (1000,))
    assert f.min() >= 0.0 and f.max() < 1.0
    z = orc.rng_normal(6, (20000,))
    assert abs(z.mean()) < 0.03 and abs(z.std() - 1.0) < 0.03
    k = orc.rng_bounded(7, 10000, 16)
    assert k.min() == 0 and k.max() == 15


def test_mla_forward_backward_smoke():
    # src/transformer.rs:1228-1266: dim16/h2/r8/rope4/dv8, x[1,3,16] LCG(-0.1,0.1,123): shape + grads flow
    cfg = om.MLAConfig(16, 2, 8, 4, 8, 10)
    W = om.mla_init_lcg(cfg, 42)
    x = orc.lcg_rand((1, 3, 16), -0.1, 0.1, 123)
    out, cache = om.mla_forward(x, W, cfg, return_cache=True)
    assert out.shape == (1, 3, 16)
    g = np.full_like(out, 1.0 / out.size)                    # loss = mean(out)
    dx, dW = om.mla_backward(g, W, cfg, cache)
    assert abs(dW["dkv"].sum()) > 0.0 and abs(dW["uk"].sum()) > 0.0


def test_rope_and_rmsnorm_backward_flow():
    # src/transformer.rs:1269-1299
    cosv, sinv = orc.rope_table(4, 10)
    x = orc.lcg_rand((1, 2, 4), -1.0, 1.0, 123)
    dx = orc.rope(np.ones_like(x), cosv, sinv, 0, backward=True)
    assert np.any(np.abs(dx) > 1e-6)
    x = orc.lcg_rand((2, 4), 0.1, 1.0, 123)
    y, rms, xh = orc.rmsnorm_fwd(x, np.ones(4), 1e-5)
    dx, dw = orc.rmsnorm_bwd(np.ones_like(x), np.ones(4), rms, xh)
    assert np.any(np.abs(dx) > 1e-6) and np.any(np.abs(dw) > 1e-6)


def test_ppo_fast_slow_alignment_distribution():
    # src/sim.rs:1181-1216: ActorCritic(12345), 6 tokens flat[t*8+i] = 0.01t + 0.001i; action
    # probabilities of the autograd path vs the KV-cached path differ by L1 < 1e-6.
    pol = om.ActorCritic(12345)
    seq, dim = 6, 8
    flat = np.array([[t * 0.01 + i * 0.001 for i in range(dim)] for t in range(seq)])
    slow = pol.forward_actor(flat)

    def sm(v):
        e = np.exp(v - v.max()); return e / e.sum()
    kv = om.KVCache(pol.backbone.cfg.num_heads)
    last = None
    for t in range(seq):
        last = pol.backbone.forward_inference_step(flat[t], kv, t)
    fast = orc.linear_forward_inference(last, *pol.actor)
    assert np.abs(sm(slow) - sm(fast)).sum() < 1e-6
    # the two RoPE position conventions really differ before the softmax saturates
    slow_tok = pol.forward_actor(flat, pos_mode="token")
    assert np.abs(sm(slow_tok) - sm(fast)).sum() < 1e-6


def test_kv_cache_prune():
    # src/transformer.rs:843-874
    cfg = om.MLAConfig(64, 4, 32, 16, 16, 256)
    kv = om.KVCache(4)
    for h in range(4):
        kv.k[h] = np.arange(5 * 32, dtype=float); kv.v[h] = np.arange(5 * 16, dtype=float)
    om.prune_kv_cache(kv, cfg, 3)
    assert kv.k[0].size == 3 * 32 and kv.k[0][0] == 64.0 and kv.v[0].size == 3 * 16 and kv.v[0][0] == 32.0


def test_gae_hand_computed_three_steps():
    # src/ppo.rs:650-671 on a three-step buffer whose middle step ends an episode, against the formulas written out
    r = np.array([1.0, 2.0, -1.0]); v = np.array([0.5, 0.25, 0.125]); term = np.array([0, 1, 0])
    adv, ret = orc.gae(r, v, term, 0.0, 1.0)
    d = 1.0 + 1e-8
    g2 = -1.0 / d + 0.0 - 0.125                      # last step: V[len] = 0
    g1 = 2.0 / d - 0.25                              # terminal: no bootstrap, no carry from g2
    g0 = 1.0 / d + 0.99 * 0.25 - 0.5 + 0.99 * 0.95 * g1
    assert np.allclose(adv, [g0, g1, g2], rtol=0, atol=1e-15) and np.allclose(ret, adv + v, rtol=0, atol=1e-15)
    adv_c, _ = orc.gae(np.array([1000.0, -1000.0]), np.zeros(2), np.array([1, 1]), 0.0, 1.0)
    assert adv_c.tolist() == [10.0, -10.0]           # normalised rewards are clipped to +-10 (:655)


def test_running_mean_std_matches_reference_formulas():
    # src/ppo.rs:444-480: count 1e-4, mean 0, var 1; one-sample updates
    rms = orc.RunningMeanStd()
    count, mean, var = 1e-4, 0.0, 1.0
    for x in (1.0, 2.0, 3.0, -4.5):
        rms.update(x)
        delta = x - mean; tot = count + 1.0
        m2 = var * count + delta ** 2 * count / tot
        mean, var, count = mean + delta / tot, m2 / tot, tot
        assert abs(rms.mean.value - mean) < 1e-15 and abs(rms.var.value - var) < 1e-15 and rms.count.value == count
    assert abs(rms.normalize(2.0) - (2.0 - mean) / (math.sqrt(var) + 1e-8)) < 1e-15
