"""GPU parity: every kernel behind the C ABI against the CPU oracle on the same seeded inputs."""
import math

import numpy as np
import pytest

import oracle as orc
from oracle import model as om
from gpu_util import TOL, dev, host, max_err, normal, rel_err, uniform, xavier

pytestmark = pytest.mark.gpu

_keep = []


def dptr(talos, a):
    """Device pointer of a fresh copy of `a`; the tensor is kept alive so that two temporaries
    passed to one call can never share memory."""
    t = dev(a); _keep.append(t)
    if len(_keep) > 64: del _keep[:32]
    return talos.ptr(t)


@pytest.fixture(scope="module")
def ctx(talos):
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    c = talos.torch_context(0)
    yield c
    c.synchronize()


def gemm(talos, ctx, opA, opB, A, B, mode, C0=None, epi=None, ldpad=0):
    import torch
    M = A.shape[0] if opA == 0 else A.shape[1]; K = A.shape[1] if opA == 0 else A.shape[0]
    N = B.shape[1] if opB == 0 else B.shape[0]

    def padded(a):
        if ldpad == 0: return dev(a), a.shape[1]
        buf = torch.full((a.shape[0], a.shape[1] + ldpad), 7.0, device="cuda:0"); buf[:, :a.shape[1]] = dev(a)
        return buf, a.shape[1] + ldpad
    a, lda = padded(A); b, ldb = padded(B)
    c = torch.full((M, N + ldpad), -123.0, device="cuda:0")
    if C0 is not None: c[:, :N] = dev(C0)
    talos.lib.talos_gemm(ctx.handle, opA, opB, M, N, K, talos.ptr(a), lda, talos.ptr(b), ldb, talos.ptr(c), N + ldpad, mode,
                         None if epi is None else __import__("ctypes").byref(epi))
    ctx.synchronize()
    if ldpad: assert torch.all(c[:, N:] == -123.0), "GEMM wrote into the leading-dimension padding"
    return c[:, :N]


def ref_gemm(opA, opB, A, B):
    return (A.T if opA else A) @ (B.T if opB else B)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_config1_gemm_512_all_forms(talos, ctx, mode):
    # benchmark configuration 1: 512^3, uniform[-1,1) seeds 42/123, A.B, A.B^T, A^T.B
    A = uniform(42, (512, 512)); B = uniform(123, (512, 512))
    for opA, opB in [(0, 0), (0, 1), (1, 0)]:
        got = gemm(talos, ctx, opA, opB, A, B, mode)
        if (opA, opB) == (0, 0):
            ref = orc.matmul(A, B)
        elif (opA, opB) == (0, 1):       # dLHS = G.B^T form (src/autograd.rs:275-308)
            ref = orc.matmul_bwd(np.zeros((512, 512)), B, A, need_dB=False)[0]
        else:                            # dRHS = A^T.G form (src/autograd.rs:310-350)
            ref = orc.matmul_bwd(A, np.zeros((512, 512)), B, need_dA=False)[1]
        assert rel_err(got, ref) <= TOL[mode], (mode, opA, opB, rel_err(got, ref))


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_odd_shapes_all_ops(talos, ctx, mode):
    sizes = [1, 3, 17, 63, 65, 127, 129]
    k = 0
    for M in sizes:
        for N in (sizes[(k + 2) % 7], sizes[(k + 5) % 7]):
            K = sizes[(k + 3) % 7]; k += 1
            for opA in (0, 1):
                for opB in (0, 1):
                    A = normal(100 + k, (K, M) if opA else (M, K)); B = normal(200 + k, (N, K) if opB else (K, N))
                    got = gemm(talos, ctx, opA, opB, A, B, mode, ldpad=3)
                    ref = ref_gemm(opA, opB, A, B)
                    assert max_err(got, ref) <= 4 * TOL[mode], (M, N, K, opA, opB, max_err(got, ref))


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_aligned_rect_shapes(talos, ctx, mode):
    for (M, N, K) in [(256, 128, 64), (384, 256, 96), (1024, 16, 256), (128, 512, 1024), (4096, 256, 64), (640, 320, 200), (600, 512, 1056), (256, 1152, 1024)]:  # the last one has a B operand too large for the pre-split / pre-round path
        for opA, opB in [(0, 0), (0, 1), (1, 0), (1, 1)]:
            A = normal(M + K, (K, M) if opA else (M, K)); B = normal(N + K + 1, (N, K) if opB else (K, N))
            got = gemm(talos, ctx, opA, opB, A, B, mode)
            assert rel_err(got, ref_gemm(opA, opB, A, B)) <= TOL[mode], (M, N, K, opA, opB)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_split_k_dw_shape_and_determinism(talos, ctx, mode):
    import torch
    # the dW shape: small output, reduction over the batch
    X = normal(7, (16384, 64)); G = normal(8, (16384, 256)); C0 = normal(9, (64, 256))
    epi = talos.Epilogue(beta=1)
    got = gemm(talos, ctx, 1, 0, X, G, mode, C0=C0, epi=epi)
    ref = C0 + X.T @ G                                  # `+=` accumulation (src/autograd.rs:346)
    assert rel_err(got, ref) <= TOL[mode]
    again = gemm(talos, ctx, 1, 0, X, G, mode, C0=C0, epi=epi)
    assert torch.equal(got, again), "split-K reduction must be bit-reproducible"


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_epilogue_bias_act_aux(talos, ctx, mode):
    import torch
    M, N, K = 300, 256, 64
    A = normal(1, (M, K)); B = xavier(2, K, N); bias = normal(3, (N,), 0.1)
    for act in ("relu", "tanh", "silu"):
        z = torch.empty(M, N, device="cuda:0"); b = dev(bias)
        epi = talos.Epilogue(bias=talos.ptr(b), aux_out=talos.ptr(z), ld_aux_out=N, act=talos.ACTS[act])
        y = gemm(talos, ctx, 0, 0, A, B, mode, epi=epi)
        zr = orc.bias_add(orc.matmul(A, B), bias)
        assert rel_err(z, zr) <= TOL[mode] and rel_err(y, om.act_fwd(zr, act)) <= TOL[mode], act
        # derivative epilogue: C = (A.B) * act'(saved)
        saved = zr if act == "silu" else om.act_fwd(zr, act)
        s = dev(saved)
        epi2 = talos.Epilogue(aux_in=talos.ptr(s), ld_aux_in=N, dact=talos.ACTS[act])
        got = gemm(talos, ctx, 0, 0, A, B, mode, epi=epi2)
        ref = om.act_bwd(orc.matmul(A, B), orc.f32r(zr), orc.f32r(om.act_fwd(zr, act)), act)
        assert rel_err(got, ref) <= max(TOL[mode], 2e-5), act


def test_grad_check_matmul_kat(talos, ctx):
    # src/grad_check.rs:30-63 through the three GEMM forms
    A = np.array([[2.0, 3.0], [4.0, 5.0]]); x = np.array([[1.0], [2.0]]); g = np.ones((2, 1))
    for mode in (0, 1, 2):
        assert np.array_equal(host(gemm(talos, ctx, 0, 0, A, x, mode)).ravel(), [8.0, 14.0])
        assert np.allclose(host(gemm(talos, ctx, 1, 0, A, g, mode)).ravel(), [6.0, 8.0], atol=1e-6)
        assert np.allclose(host(gemm(talos, ctx, 0, 1, g, x, mode)).ravel(), [1.0, 2.0, 1.0, 2.0], atol=1e-6)


def test_gemm_empty_and_errors(talos, ctx):
    import torch
    a = torch.zeros(4, 4, device="cuda:0")
    talos.lib.talos_gemm(ctx.handle, 0, 0, 0, 4, 4, talos.ptr(a), 4, talos.ptr(a), 4, talos.ptr(a), 4, 0, None)   # M = 0: no-op
    c = torch.full((4, 4), 5.0, device="cuda:0")
    talos.lib.talos_gemm(ctx.handle, 0, 0, 4, 4, 0, talos.ptr(a), 4, talos.ptr(a), 4, talos.ptr(c), 4, 0, None)   # K = 0: C = 0
    ctx.synchronize(); assert torch.all(c == 0.0)
    with pytest.raises(talos.TalosError) as e:
        talos.lib.talos_gemm(ctx.handle, 0, 0, 4, 4, 4, talos.ptr(a), 2, talos.ptr(a), 4, talos.ptr(c), 4, 0, None)
    assert e.value.status == talos.ERR_SHAPE and "dimension mismatch" in str(e.value)
    with pytest.raises(talos.TalosError) as e:
        talos.lib.talos_gemm(ctx.handle, 0, 0, 4, 4, 4, None, 4, talos.ptr(a), 4, talos.ptr(c), 4, 0, None)
    assert e.value.status == talos.ERR_ARG


def test_gemm_batched_qkt_and_pv(talos, ctx):
    import torch
    BH, S, D, Dv = 37, 48, 24, 20
    q = normal(1, (BH, S, D)); k = normal(2, (BH, S, D)); v = normal(3, (BH, S, Dv))
    sc = torch.empty(BH, S, S, device="cuda:0"); dq, dk, dv = dev(q), dev(k), dev(v)
    talos.lib.talos_gemm_batched(ctx.handle, 0, 1, S, S, D, talos.ptr(dq), D, S * D, talos.ptr(dk), D, S * D, talos.ptr(sc), S, S * S, BH, 0, 0)
    ctx.synchronize()
    ref = orc.bmm_qkt(q, k)
    assert rel_err(sc, ref) <= 1e-5
    p = orc.f32r(orc.softmax(ref)); dp = dev(p); out = torch.empty(BH, S, Dv, device="cuda:0")
    talos.lib.talos_gemm_batched(ctx.handle, 0, 0, S, Dv, S, talos.ptr(dp), S, S * S, talos.ptr(dv), Dv, S * Dv, talos.ptr(out), Dv, S * Dv, BH, 0, 0)
    ctx.synchronize()
    assert rel_err(out, orc.bmm_pv(p, v)) <= 1e-5


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_config2_mlp_forward_backward(talos, ctx, mode):
    import torch
    # benchmark configuration 2: batch 8192, 64 -> 256 -> 256 -> 16, tanh, Xavier-uniform, N(0,1) inputs and upstream grad
    n = 8192; dims = [64, 256, 256, 16]; acts = ["tanh", "tanh", "none"]
    X = normal(1, (n, 64)); dY = normal(5, (n, 16))
    Ws = [xavier(2 + i, dims[i], dims[i + 1]) for i in range(3)]
    for bias_std in (0.0, 0.1):
        bs = [normal(20 + i, (dims[i + 1],), bias_std) if bias_std else np.zeros(dims[i + 1]) for i in range(3)]
        zs, hs = om.mlp_fwd(X, Ws, bs, acts)
        rdx, rdW, rdb = om.mlp_bwd(X, Ws, bs, acts, zs, hs, dY)
        x = dev(X); w = [dev(W) for W in Ws]; b = [dev(v) for v in bs]
        h = [torch.empty(n, d, device="cuda:0") for d in dims[1:]]
        inp = x
        for l in range(3):
            talos.lib.talos_linear_fwd(ctx.handle, talos.ptr(inp), talos.ptr(w[l]), talos.ptr(b[l]), talos.ptr(h[l]), None, n,
                                       dims[l], dims[l + 1], talos.ACTS[acts[l]], mode)
            inp = h[l]
        g = dev(dY)
        dW = [torch.empty_like(v) for v in w]; db = [torch.empty_like(v) for v in b]
        for l in (2, 1, 0):
            dx = torch.empty(n, dims[l], device="cuda:0")
            talos.lib.talos_linear_bwd(ctx.handle, talos.ptr(x if l == 0 else h[l - 1]), talos.ptr(w[l]), talos.ptr(h[l]), talos.ptr(g),
                                       talos.ptr(dx), talos.ptr(dW[l]), talos.ptr(db[l]), n, dims[l], dims[l + 1],
                                       talos.ACTS[acts[l]], mode, 0)
            g = dx
        ctx.synchronize()
        tol = TOL[mode]
        assert rel_err(h[2], hs[2]) <= tol and rel_err(g, rdx) <= 1.5 * tol
        for l in range(3):
            assert rel_err(dW[l], rdW[l]) <= 1.5 * tol, (l, rel_err(dW[l], rdW[l]))
            assert rel_err(db[l], rdb[l]) <= 1.5 * tol, (l, rel_err(db[l], rdb[l]))
        # identical argmax actions on the 16-way head (rows whose top-2 oracle gap < 1e-6 * scale are exempt)
        top2 = np.sort(hs[2], axis=1)[:, -2:]; safe = (top2[:, 1] - top2[:, 0]) > (1e-5 if mode != 2 else 1e-2)
        assert np.array_equal(host(h[2]).argmax(1)[safe], hs[2].argmax(1)[safe])
        assert safe.mean() > 0.9


def test_linear_bwd_accumulates(talos, ctx):
    import torch
    n, fi, fo = 100, 12, 20
    X = normal(1, (n, fi)); W = normal(2, (fi, fo)); dY = normal(3, (n, fo))
    dx0 = normal(4, (n, fi)); dW0 = normal(5, (fi, fo)); db0 = normal(6, (fo,))
    dx, dW, db = dev(dx0), dev(dW0), dev(db0)
    talos.lib.talos_linear_bwd(ctx.handle, dptr(talos, X), dptr(talos, W), None, dptr(talos, dY), talos.ptr(dx), talos.ptr(dW),
                               talos.ptr(db), n, fi, fo, 0, 0, 7)
    ctx.synchronize()
    assert rel_err(dx, dx0 + dY @ W.T) <= 1e-5 and rel_err(dW, dW0 + X.T @ dY) <= 1e-5 and rel_err(db, db0 + dY.sum(0)) <= 1e-5


def test_bias_add_colsum(talos, ctx):
    import torch
    for rows, n in [(1, 1), (2, 1), (777, 33), (8192, 256), (5, 1000)]:
        Y = normal(1, (rows, n)); b = normal(2, (n,))
        y = dev(Y); talos.lib.talos_bias_add(ctx.handle, talos.ptr(y), dptr(talos, b), rows, n)
        out = dev(np.ones(n)); talos.lib.talos_colsum(ctx.handle, dptr(talos, Y), talos.ptr(out), rows, n, 1)
        ctx.synchronize()
        assert rel_err(y, orc.bias_add(Y, b)) <= 1e-6
        assert max_err(out, 1.0 + orc.bias_bwd(Y, n)) <= 1e-5
    # src/grad_check.rs:66-90
    y = dev(np.array([[1.0], [2.0]])); talos.lib.talos_bias_add(ctx.handle, talos.ptr(y), dptr(talos, np.array([10.0])), 2, 1)
    o = dev(np.zeros(1)); talos.lib.talos_colsum(ctx.handle, dptr(talos, np.ones((2, 1))), talos.ptr(o), 2, 1, 0)
    ctx.synchronize()
    assert host(y).ravel().tolist() == [11.0, 12.0] and host(o)[0] == 2.0


def test_rmsnorm_fwd_bwd(talos, ctx):
    import torch
    for rows, dim, eps in [(1, 4, 1e-5), (2, 4, 1e-5), (1000, 64, 1e-5), (4096, 256, 1e-6), (333, 512, 1e-6), (50, 257, 1e-5), (7, 1024, 1e-6), (3, 1100, 1e-5)]:
        X = normal(rows + dim, (rows, dim)); gam = 1.0 + normal(3, (dim,), 0.1); G = normal(4, (rows, dim))
        y = torch.empty(rows, dim, device="cuda:0"); inv = torch.empty(rows, device="cuda:0"); x = dev(X); g = dev(gam)
        talos.lib.talos_rmsnorm_fwd(ctx.handle, talos.ptr(x), talos.ptr(g), eps, rows, dim, talos.ptr(y), talos.ptr(inv))
        ry, rrms, rxh = orc.rmsnorm_fwd(X, gam, eps)
        ctx.synchronize()
        assert rel_err(y, ry) <= 1e-6 and rel_err(inv, 1.0 / rrms) <= 1e-6, (rows, dim)
        dx0 = normal(5, (rows, dim)); dg0 = normal(6, (dim,))
        dx = dev(dx0); dg = dev(dg0)
        talos.lib.talos_rmsnorm_bwd(ctx.handle, dptr(talos, G), talos.ptr(x), talos.ptr(g), talos.ptr(inv), rows, dim, talos.ptr(dx), talos.ptr(dg), 3)
        rdx, rdw = orc.rmsnorm_bwd(G, gam, rrms, rxh)
        ctx.synchronize()
        assert rel_err(dx, dx0 + rdx) <= 1e-5 and rel_err(dg, dg0 + rdw) <= 1e-5, (rows, dim)
        dx2 = torch.empty(rows, dim, device="cuda:0")
        talos.lib.talos_rmsnorm_bwd(ctx.handle, dptr(talos, G), talos.ptr(x), talos.ptr(g), talos.ptr(inv), rows, dim, talos.ptr(dx2), None, 0)
        ctx.synchronize()
        assert rel_err(dx2, rdx) <= 1e-5


def test_rope_both_conventions(talos, ctx):
    import torch
    B, S, H, dr, maxlen = 3, 10, 4, 16, 12
    cosv, sinv = orc.rope_table(dr, maxlen)
    c = torch.empty(maxlen * dr // 2, device="cuda:0"); s = torch.empty_like(c)
    talos.lib.talos_rope_table(ctx.handle, dr, maxlen, 10000.0, talos.ptr(c), talos.ptr(s))
    assert np.array_equal(host(c), orc.f32r(cosv)) and np.array_equal(host(s), orc.f32r(sinv))
    cosf, sinf = orc.f32r(cosv), orc.f32r(sinv)
    X = normal(1, (B, S, H, dr)); x = dev(X); y = torch.empty_like(x)
    # TOKEN: rotate by token position
    talos.lib.talos_rope(ctx.handle, talos.ptr(x), talos.ptr(y), talos.ptr(c), talos.ptr(s), c.numel(), B, S, H, dr, 0, 0, 0)
    ctx.synchronize(); assert rel_err(y, orc.rope_token(X, cosf, sinf, 0)) <= 1e-6
    # start_pos pushes the last tokens past the table: they stay unrotated (src/transformer.rs:586-588)
    talos.lib.talos_rope(ctx.handle, talos.ptr(x), talos.ptr(y), talos.ptr(c), talos.ptr(s), c.numel(), B, S, H, dr, 5, 0, 0)
    ctx.synchronize(); ref = orc.rope_token(X, cosf, sinf, 5)
    assert rel_err(y, ref) <= 1e-6 and np.array_equal(host(y)[:, 7:], X[:, 7:])
    # HEAD_INDEX: what RoPE::forward does to [B,S,H,dr] on the autograd path (src/transformer.rs:262)
    talos.lib.talos_rope(ctx.handle, talos.ptr(x), talos.ptr(y), talos.ptr(c), talos.ptr(s), c.numel(), B * S, H, 1, dr, 0, 0, 0)
    ctx.synchronize(); assert rel_err(y, orc.rope(X, cosf, sinf, 0)) <= 1e-6
    # backward = transposed rotation, accumulating (src/transformer.rs:319-331)
    G = normal(2, X.shape); acc0 = normal(3, X.shape); acc = dev(acc0)
    talos.lib.talos_rope(ctx.handle, dptr(talos, G), talos.ptr(acc), talos.ptr(c), talos.ptr(s), c.numel(), B * S, H, 1, dr, 0, 1, 1)
    ctx.synchronize(); assert rel_err(acc, acc0 + orc.rope(G, cosf, sinf, 0, backward=True)) <= 1e-6


def test_softmax_fwd_bwd(talos, ctx):
    import torch
    for rows, n, causal in [(1, 1, 0), (64, 64, 0), (8 * 64, 64, 64), (300, 128, 0), (256, 128, 128), (17, 5, 0), (40, 200, 0), (9, 1000, 0)]:
        X = normal(rows + n, (rows, n), 2.0); scale = 1.0 / math.sqrt(96.0)
        y = torch.empty(rows, n, device="cuda:0")
        talos.lib.talos_softmax_fwd(ctx.handle, dptr(talos, X), talos.ptr(y), rows, n, scale, causal)
        ref = orc.softmax(orc.f32r(X) * np.float64(np.float32(scale)), causal)
        ctx.synchronize()
        assert rel_err(y, ref) <= 2e-6, (rows, n, causal)
        G = normal(5, (rows, n)); dx0 = normal(6, (rows, n)); dx = dev(dx0)
        talos.lib.talos_softmax_bwd(ctx.handle, dptr(talos, ref), dptr(talos, G), talos.ptr(dx), rows, n, scale, 1)
        ctx.synchronize()
        yr = orc.f32r(ref)
        assert rel_err(dx, dx0 + np.float64(np.float32(scale)) * orc.softmax_bwd(yr, G)) <= 1e-5
    talos.lib.talos_softmax_fwd(ctx.handle, None, None, 5, 0, 1.0, 0)        # empty rows: nothing to do


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_attention_fwd_bwd(talos, ctx, mode):
    import torch
    tol = TOL[mode]
    # (6,128,96,64) is the MLA shape of config 4, (16,64,32,32) the block of config 3; the ragged ones fall back to
    # the fused CUDA-core kernel (forward) / the fp32 batched GEMM (backward) in every mode.
    for BH, S, dqk, dv, causal in [(5, 3, 12, 8, 0), (16, 64, 32, 32, 1), (6, 128, 96, 64, 0), (3, 100, 40, 24, 0), (4, 17, 8, 130 - 2, 1), (300, 16, 32, 16, 0)]:
        q = normal(1, (BH, S, dqk)); k = normal(2, (BH, S, dqk)); v = normal(3, (BH, S, dv)); scale = 1.0 / math.sqrt(dqk)
        sc = orc.bmm_qkt(q, k) * np.float64(np.float32(scale))
        P = orc.softmax(sc, S if causal else 0); O = orc.bmm_pv(P, v)
        out = torch.empty(BH, S, dv, device="cuda:0"); probs = torch.empty(BH, S, S, device="cuda:0")
        dq_, dk_, dv_ = dev(q), dev(k), dev(v)
        talos.lib.talos_attention_fwd(ctx.handle, talos.ptr(dq_), talos.ptr(dk_), talos.ptr(dv_), talos.ptr(out), talos.ptr(probs), BH, S, dqk, dv, scale, causal, mode)
        ctx.synchronize()
        assert rel_err(probs, P) <= tol and rel_err(out, O) <= tol, (BH, S, rel_err(probs, P), rel_err(out, O))
        out2 = torch.empty_like(out)                      # without the probabilities: scores go through scratch
        talos.lib.talos_attention_fwd(ctx.handle, talos.ptr(dq_), talos.ptr(dk_), talos.ptr(dv_), talos.ptr(out2), None, BH, S, dqk, dv, scale, causal, mode)
        ctx.synchronize()
        assert torch.equal(out, out2), (BH, S)
        G = normal(4, (BH, S, dv))
        gq = torch.empty_like(dq_); gk = torch.empty_like(dk_); gv = torch.empty_like(dv_)
        talos.lib.talos_attention_bwd(ctx.handle, talos.ptr(dq_), talos.ptr(dk_), talos.ptr(dv_), talos.ptr(probs), dptr(talos, G),
                                      talos.ptr(gq), talos.ptr(gk), talos.ptr(gv), BH, S, dqk, dv, scale, mode)
        ctx.synchronize()
        dP, rdv = orc.bmm_pv_bwd(P, v, G)
        dS = orc.softmax_bwd(P, dP) * np.float64(np.float32(scale))
        rdq, rdk = orc.bmm_qkt_bwd(q, k, dS)
        assert rel_err(gq, rdq) <= 2 * tol and rel_err(gk, rdk) <= 2 * tol and rel_err(gv, rdv) <= 2 * tol, (BH, S, rel_err(gq, rdq), rel_err(gk, rdk), rel_err(gv, rdv))


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_batched_all_ops(talos, ctx, mode):
    import torch
    # R12 shapes (src/transformer.rs:877-1050) plus ragged ones; beta=1 accumulates into C
    for batch, M, N, K in [(7, 64, 64, 32), (5, 128, 64, 128), (3, 72, 88, 104), (9, 33, 20, 12), (130, 16, 16, 16)]:
        for opA, opB in [(0, 0), (0, 1), (1, 0), (1, 1)]:
            A = normal(10 + M, (batch, K, M) if opA else (batch, M, K)); B = normal(20 + N, (batch, N, K) if opB else (batch, K, N))
            C0 = normal(30, (batch, M, N))
            a, b = dev(A), dev(B)
            for beta in (0, 1):
                c = dev(C0)
                talos.lib.talos_gemm_batched(ctx.handle, opA, opB, M, N, K, talos.ptr(a), A.shape[2], A.shape[1] * A.shape[2],
                                             talos.ptr(b), B.shape[2], B.shape[1] * B.shape[2], talos.ptr(c), N, M * N, batch, beta, mode)
                ctx.synchronize()
                ref = np.einsum("bmk,bkn->bmn", np.swapaxes(A, 1, 2) if opA else A, np.swapaxes(B, 1, 2) if opB else B) + (C0 if beta else 0)
                assert rel_err(c, ref) <= TOL[mode], (batch, M, N, K, opA, opB, beta, rel_err(c, ref))


def test_gae_and_advantage_normalisation(talos, ctx):
    import torch
    # lengths around the 2 048-element scan chunk and a rollout-sized buffer; episode ends every ~50 steps
    for n in (1, 7, 2047, 2048, 2049, 50000, 1048576):
        r = orc.f32r(orc.rng_normal(70, (n,)) * 3.0 + 1.0); v = orc.f32r(orc.rng_normal(71, (n,)))
        term = (orc.rng_bounded(72, n, 50) == 0).astype(np.int32)
        rms = orc.RunningMeanStd(); rms.update(r[:min(n, 4096)])
        mean, var = float(np.float32(rms.mean.value)), float(np.float32(rms.var.value))
        adv_ref, ret_ref = orc.gae(r, v, term, mean, var)
        d_r, d_v = dev(r), dev(v); d_t = torch.from_numpy(term).cuda()
        adv = torch.empty(n, device="cuda:0"); ret = torch.empty(n, device="cuda:0")
        talos.lib.talos_gae(ctx.handle, talos.ptr(d_r), talos.ptr(d_v), talos.ptr(d_t), n, 0.99, 0.95, mean, var, talos.ptr(adv), talos.ptr(ret))
        ctx.synchronize()
        assert rel_err(adv, adv_ref) <= 1e-5 and rel_err(ret, ret_ref) <= 1e-5, (n, rel_err(adv, adv_ref))
        if n > 1:
            m = orc.sum_f64(adv_ref) / n; sd = math.sqrt(orc.sum_sq_diff(adv_ref, m) / n) + 1e-8
            norm_ref = orc.normalize_slice(adv_ref, m, sd)
            stats = torch.empty(2, device="cuda:0")
            talos.lib.talos_normalize_slice(ctx.handle, talos.ptr(adv), n, talos.ptr(adv), talos.ptr(stats))      # in place
            ctx.synchronize()
            assert rel_err(adv, norm_ref) <= 1e-5, (n, rel_err(adv, norm_ref))
            st = host(stats); assert abs(st[0] - m) <= 1e-5 * max(1.0, abs(m)) + 1e-6 and abs(st[1] - sd) <= 1e-5 * sd
    # no episode boundary at all and all boundaries: the two extremes of the recurrence
    n = 5000; r = orc.f32r(orc.rng_normal(73, (n,))); v = orc.f32r(orc.rng_normal(74, (n,)))
    for term in (np.zeros(n, np.int32), np.ones(n, np.int32)):
        adv_ref, ret_ref = orc.gae(r, v, term, 0.0, 1.0)
        d_r, d_v = dev(r), dev(v); d_t = torch.from_numpy(term).cuda()
        adv = torch.empty(n, device="cuda:0"); ret = torch.empty(n, device="cuda:0")
        talos.lib.talos_gae(ctx.handle, talos.ptr(d_r), talos.ptr(d_v), talos.ptr(d_t), n, 0.99, 0.95, 0.0, 1.0, talos.ptr(adv), talos.ptr(ret))
        ctx.synchronize()
        assert rel_err(adv, adv_ref) <= 1e-5 and rel_err(ret, ret_ref) <= 1e-5
    talos.lib.talos_gae(ctx.handle, None, None, None, 0, 0.99, 0.95, 0.0, 1.0, None, None)                       # empty rollout: nothing to do
    # buffers that start one element into an allocation: not 16-byte aligned, the element-wise load path
    n = 4500; r = orc.f32r(orc.rng_normal(75, (n,))); v = orc.f32r(orc.rng_normal(76, (n,))); term = (orc.rng_bounded(77, n, 9) == 0).astype(np.int32)
    adv_ref, ret_ref = orc.gae(r, v, term, 0.25, 2.0)
    pad = lambda a, dt: torch.cat([torch.zeros(1, dtype=dt), torch.from_numpy(a).to(dt)]).cuda()[1:]
    d_r, d_v, d_t = pad(r, torch.float32), pad(v, torch.float32), pad(term, torch.int32)
    adv = torch.empty(n + 1, device="cuda:0")[1:]; ret = torch.empty(n + 1, device="cuda:0")[1:]
    talos.lib.talos_gae(ctx.handle, talos.ptr(d_r), talos.ptr(d_v), talos.ptr(d_t), n, 0.99, 0.95, 0.25, 2.0, talos.ptr(adv), talos.ptr(ret))
    out = torch.empty(n + 1, device="cuda:0")[1:]
    talos.lib.talos_normalize_slice(ctx.handle, talos.ptr(adv), n, talos.ptr(out), None)
    ctx.synchronize()
    assert rel_err(adv, adv_ref) <= 1e-5 and rel_err(ret, ret_ref) <= 1e-5
    m = orc.sum_f64(adv_ref) / n; sd = math.sqrt(orc.sum_sq_diff(adv_ref, m) / n) + 1e-8
    assert rel_err(out, orc.normalize_slice(adv_ref, m, sd)) <= 1e-5


def test_dqn_step_pieces(talos, ctx):
    import torch
    for B, A in [(64, 5), (1, 5), (1000, 3), (37, 16)]:          # 64 x 5 is the crate's batch (src/dqn.rs:34, :15)
        v = orc.f32r(orc.rng_normal(80, (B, 1))); adv = orc.f32r(orc.rng_normal(81, (B, A)))
        q = torch.empty(B, A, device="cuda:0")
        talos.lib.talos_dueling_combine_fwd(ctx.handle, dptr(talos, v), dptr(talos, adv), talos.ptr(q), B, A)
        ctx.synchronize()
        q_ref = om.dueling_combine(v, adv)
        assert max_err(q, q_ref) <= 1e-6
        g = orc.f32r(orc.rng_normal(82, (B, A))); dv0 = orc.f32r(orc.rng_normal(83, (B, 1))); da0 = orc.f32r(orc.rng_normal(84, (B, A)))
        dv_ref, da_ref = om.dueling_combine_bwd(g)
        for acc in (0, 1):
            dv = dev(dv0); da = dev(da0)
            talos.lib.talos_dueling_combine_bwd(ctx.handle, dptr(talos, g), talos.ptr(dv), talos.ptr(da), B, A, acc)
            ctx.synchronize()
            assert max_err(dv, dv_ref + acc * dv0) <= 2e-6 and max_err(da, da_ref + acc * da0) <= 2e-6
        qe = orc.f32r(orc.rng_normal(85, (B, A))); qt = orc.f32r(orc.rng_normal(86, (B, A)))
        qe[0, :] = qe[0, 0]                                       # a tie: the first maximum must win
        r = orc.f32r(orc.rng_normal(87, (B,))); done = (orc.rng_bounded(88, B, 4) == 0).astype(np.float64)
        tgt = torch.empty(B, device="cuda:0")
        talos.lib.talos_dqn_target(ctx.handle, dptr(talos, qe), dptr(talos, qt), dptr(talos, r), dptr(talos, done), 0.99, talos.ptr(tgt), B, A)
        ctx.synchronize()
        t_ref = om.dqn_target(qe, qt, r, done, np.float64(np.float32(0.99)))
        assert max_err(tgt, t_ref) <= 1e-6
        acts = orc.rng_bounded(89, B, A).astype(np.int32); d_acts = torch.from_numpy(acts).cuda()
        loss = torch.empty(1, device="cuda:0"); dq = torch.full((B, A), 7.0, device="cuda:0")
        talos.lib.talos_dqn_loss_fwd_bwd(ctx.handle, talos.ptr(q), talos.ptr(d_acts), talos.ptr(tgt), talos.ptr(loss), talos.ptr(dq), B, A)
        ctx.synchronize()
        l_ref, dq_ref = om.dqn_loss_fwd_bwd(q_ref, acts, t_ref)
        assert abs(host(loss)[0] - l_ref) <= 1e-5 * max(1.0, abs(l_ref)) and max_err(dq, dq_ref) <= 1e-6 * max(1.0, np.abs(dq_ref).max())
    n = 70000; t0 = orc.f32r(orc.rng_normal(90, (n,))); s0 = orc.f32r(orc.rng_normal(91, (n,)))
    t = dev(t0)
    talos.lib.talos_soft_update(ctx.handle, talos.ptr(t), dptr(talos, s0), 0.005, n)
    ctx.synchronize()
    assert max_err(t, om.soft_update(t0, s0, np.float64(np.float32(0.005)))) <= 1e-6


def test_layout_ops(talos, ctx):
    import ctypes as C
    import torch
    # src/transformer.rs:1212-1225
    t = dev(np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])); o = torch.empty(3, 2, device="cuda:0")
    talos.lib.talos_transpose(ctx.handle, talos.ptr(t), talos.ptr(o), (C.c_int64 * 2)(2, 3), 2, 0, 1, 0)
    ctx.synchronize(); assert host(o).ravel().tolist() == [1, 4, 2, 5, 3, 6]
    for shape, d0, d1 in [((2, 5, 3, 7), 1, 2), ((4, 6, 5), 0, 2), ((3, 4, 5, 2, 3), 1, 3), ((33, 70), 0, 1), ((2, 3, 40, 33), 2, 3), ((9,), 0, 0)]:
        X = normal(1, shape); x = dev(X)
        oshape = list(shape); oshape[d0], oshape[d1] = oshape[d1], oshape[d0]
        y = torch.empty(oshape, device="cuda:0")
        talos.lib.talos_transpose(ctx.handle, talos.ptr(x), talos.ptr(y), (C.c_int64 * len(shape))(*shape), len(shape), d0, d1, 0)
        ctx.synchronize(); assert np.array_equal(host(y), orc.transpose(X, d0, d1)), shape
        acc0 = normal(2, oshape); acc = dev(acc0)       # backward: scatter-add of a gradient given in the transposed layout
        talos.lib.talos_transpose(ctx.handle, talos.ptr(x), talos.ptr(acc), (C.c_int64 * len(shape))(*shape), len(shape), d0, d1, 1)
        ctx.synchronize(); assert rel_err(acc, acc0 + X.swapaxes(d0, d1)) <= 1e-6
    A = normal(3, (50, 8)); B = normal(4, (50, 3)); out = torch.empty(50, 11, device="cuda:0")
    talos.lib.talos_concat_last(ctx.handle, dptr(talos, A), dptr(talos, B), talos.ptr(out), 50, 8, 3)
    ctx.synchronize(); assert np.array_equal(host(out), np.concatenate([A, B], -1))
    ga = dev(np.ones((50, 8))); gb = dev(np.ones((50, 3)))
    talos.lib.talos_split_last(ctx.handle, talos.ptr(out), talos.ptr(ga), talos.ptr(gb), 50, 8, 3, 1)
    ctx.synchronize(); assert rel_err(ga, 1 + A) <= 1e-6 and rel_err(gb, 1 + B) <= 1e-6
    X = normal(5, (4, 6, 10)); y = torch.empty(4, 10, device="cuda:0")
    talos.lib.talos_last_token(ctx.handle, dptr(talos, X), talos.ptr(y), 4, 6, 10)
    ctx.synchronize(); assert np.array_equal(host(y), X[:, -1, :])


def test_eltwise_and_reductions(talos, ctx):
    import torch
    n = 5000
    X = normal(1, (n,)); Xp = np.abs(X) + 0.1; G = normal(2, (n,))
    f = {"relu": lambda x: np.where(x > 0, x, 0), "tanh": np.tanh, "silu": lambda x: x / (1 + np.exp(-x)), "exp": np.exp, "log": np.log,
         "sin": np.sin, "cos": np.cos, "sqrt": np.sqrt, "clip": lambda x: np.clip(x, 0.8, 1.2), "neg": lambda x: -x, "scale": lambda x: x * np.float64(np.float32(0.3))}
    df = {"relu": lambda x: (x > 0) * 1.0, "tanh": lambda x: 1 - np.tanh(x) ** 2, "silu": lambda x: om.act_bwd(np.ones_like(x), x, None, "silu"),
          "exp": np.exp, "log": lambda x: 1 / x, "sin": np.cos, "cos": lambda x: -np.sin(x), "sqrt": lambda x: 0.5 / np.sqrt(x),
          "clip": lambda x: ((x >= np.float32(0.8)) & (x <= np.float32(1.2))) * 1.0, "neg": lambda x: -np.ones_like(x), "scale": lambda x: np.full_like(x, np.float64(np.float32(0.3)))}
    for name in f:
        src = Xp if name in ("log", "sqrt", "clip") else X
        p0, p1 = (0.8, 1.2) if name == "clip" else (0.3, 0.0)
        x = dev(src); y = torch.empty(n, device="cuda:0"); dx0 = normal(3, (n,)); dx = dev(dx0)
        talos.lib.talos_eltwise_unary(ctx.handle, talos.EW[name], talos.ptr(x), talos.ptr(y), n, p0, p1)
        talos.lib.talos_eltwise_unary_bwd(ctx.handle, talos.EW[name], talos.ptr(x), dptr(talos, G), talos.ptr(dx), n, p0, p1)
        ctx.synchronize()
        assert rel_err(y, f[name](src)) <= 1e-6, name
        assert rel_err(dx, dx0 + G * df[name](src)) <= 2e-6, name
    A = normal(4, (n,)); B = Xp
    for name, fn, da, db in [("add", lambda a, b: a + b, lambda a, b: 1 + 0 * a, lambda a, b: 1 + 0 * a), ("sub", lambda a, b: a - b, lambda a, b: 1 + 0 * a, lambda a, b: -1 + 0 * a),
                             ("mul", lambda a, b: a * b, lambda a, b: b, lambda a, b: a), ("div", lambda a, b: a / b, lambda a, b: 1 / b, lambda a, b: -a / b ** 2)]:
        a = dev(A); b = dev(B); y = torch.empty(n, device="cuda:0"); ga = dev(np.zeros(n)); gb = dev(np.zeros(n))
        talos.lib.talos_eltwise_binary(ctx.handle, talos.EW[name], talos.ptr(a), talos.ptr(b), talos.ptr(y), n)
        talos.lib.talos_eltwise_binary_bwd(ctx.handle, talos.EW[name], talos.ptr(a), talos.ptr(b), dptr(talos, G), talos.ptr(ga), talos.ptr(gb), n)
        ctx.synchronize()
        assert rel_err(y, fn(A, B)) <= 1e-6 and rel_err(ga, G * da(A, B)) <= 1e-6 and rel_err(gb, G * db(A, B)) <= 1e-6, name
    # src/grad_check.rs:93-114: f(x) = x^2 sin x at 2.0; the x*x node has aliased operands (src/autograd.rs:1729)
    x = dev(np.array([2.0])); xx = torch.empty(1, device="cuda:0"); sx = torch.empty(1, device="cuda:0"); yv = torch.empty(1, device="cuda:0")
    talos.lib.talos_eltwise_binary(ctx.handle, talos.EW["mul"], talos.ptr(x), talos.ptr(x), talos.ptr(xx), 1)
    talos.lib.talos_eltwise_unary(ctx.handle, talos.EW["sin"], talos.ptr(x), talos.ptr(sx), 1, 0.0, 0.0)
    talos.lib.talos_eltwise_binary(ctx.handle, talos.EW["mul"], talos.ptr(xx), talos.ptr(sx), talos.ptr(yv), 1)
    gx = dev(np.zeros(1)); gxx = dev(np.zeros(1)); gsx = dev(np.zeros(1)); one = dev(np.ones(1))
    talos.lib.talos_eltwise_binary_bwd(ctx.handle, talos.EW["mul"], talos.ptr(xx), talos.ptr(sx), talos.ptr(one), talos.ptr(gxx), talos.ptr(gsx), 1)
    talos.lib.talos_eltwise_unary_bwd(ctx.handle, talos.EW["sin"], talos.ptr(x), talos.ptr(gsx), talos.ptr(gx), 1, 0.0, 0.0)
    talos.lib.talos_eltwise_binary_bwd(ctx.handle, talos.EW["mul"], talos.ptr(x), talos.ptr(x), talos.ptr(gxx), talos.ptr(gx), talos.ptr(gx), 1)
    ctx.synchronize()
    fn = lambda v: v * v * math.sin(v)
    assert abs(host(gx)[0] - (fn(2.0 + 1e-6) - fn(2.0 - 1e-6)) / 2e-6) < 1e-4
    # sum / mean / broadcast (src/autograd.rs:443-509, :1869-1875)
    for m in (1, 7, 1000, 1 << 20):
        V = normal(9, (m,)); o = dev(np.array([2.0]))
        talos.lib.talos_reduce_sum(ctx.handle, dptr(talos, V), m, 1.0 / m, talos.ptr(o), 1)
        ctx.synchronize(); assert abs(host(o)[0] - (2.0 + V.mean())) <= 1e-5
    b = torch.empty(4, device="cuda:0"); talos.lib.talos_fill_from_scalar(ctx.handle, dptr(talos, np.array([5.0])), 1.0, talos.ptr(b), 4, 0)
    ctx.synchronize(); assert host(b).tolist() == [5.0, 5.0, 5.0, 5.0]


def test_ppo_loss_and_adam(talos, ctx):
    import torch
    for n, A, ld in [(1, 5, 5), (1000, 5, 8), (65536, 16, 32), (333, 7, 7)]:
        logits = normal(1, (n, A)); values = normal(2, (n,)); actions = orc.rng_bounded(3, n, A)
        adv = normal(4, (n,)); ret = normal(5, (n,)); old = orc.f32r(-1.6 + 0.4 * orc.rng_normal(6, (n,)))
        lbuf = torch.zeros(n, ld, device="cuda:0"); lbuf[:, :A] = dev(logits)
        dl = torch.zeros(n, ld, device="cuda:0"); dv = torch.empty(n, device="cuda:0"); stats = torch.zeros(4, device="cuda:0")
        talos.lib.talos_ppo_loss_fwd_bwd(ctx.handle, talos.ptr(lbuf), ld, dptr(talos, values), 1, dptr(talos, actions), dptr(talos, old),
                                         dptr(talos, adv), dptr(talos, ret), n, A, 0.2, 0.5, 0.01, float(n), talos.ptr(dl), ld, talos.ptr(dv), 1, talos.ptr(stats))
        ctx.synchronize()
        loss, rdl, rdv, kl = om.ppo_loss_fwd_bwd(logits, values, actions, old, adv, ret)
        st = host(stats)
        assert rel_err(dl[:, :A], rdl) <= 1e-5 and rel_err(dv, rdv) <= 1e-5, (n, A)
        assert abs(st[0] / n - loss) <= 1e-5 * max(1.0, abs(loss)) and abs(st[1] - kl) <= 1e-4 * max(1.0, abs(kl)) and st[2] == n
    n = 86801
    P = normal(1, (n,)); G = normal(2, (n,), 0.01)
    for clip in (0.0, 1.0):
        p = dev(P); m = torch.zeros(n, device="cuda:0"); v = torch.zeros(n, device="cuda:0")
        rp = [P.copy()]; rm = [np.zeros(n)]; rv = [np.zeros(n)]
        for t in range(1, 6):
            g = orc.f32r(G * t)
            talos.lib.talos_adam_step(ctx.handle, talos.ptr(p), dptr(talos, g), talos.ptr(m), talos.ptr(v), n, t, 3e-4, 0.9, 0.999, 1e-8, 1.0, clip)
            om.adam_step(rp, [g], rm, rv, t, np.float64(np.float32(3e-4)), np.float64(np.float32(0.9)), np.float64(np.float32(0.999)), np.float64(np.float32(1e-8)), clip_norm=clip or None)
        ctx.synchronize()
        assert rel_err(p, rp[0]) <= 1e-6 and rel_err(p - dev(P), rp[0] - P) <= 3e-4 and rel_err(m, rm[0]) <= 1e-5, clip


def test_run_twice_bit_equal(talos, ctx):
    import torch
    rows, dim = 5000, 256
    X = normal(1, (rows, dim)); G = normal(2, (rows, dim)); gam = np.ones(dim)
    outs = []
    for _ in range(2):
        x = dev(X); inv = torch.empty(rows, device="cuda:0"); y = torch.empty(rows, dim, device="cuda:0"); dx = torch.empty_like(y); dg = torch.empty(dim, device="cuda:0")
        talos.lib.talos_rmsnorm_fwd(ctx.handle, talos.ptr(x), dptr(talos, gam), 1e-6, rows, dim, talos.ptr(y), talos.ptr(inv))
        talos.lib.talos_rmsnorm_bwd(ctx.handle, dptr(talos, G), talos.ptr(x), dptr(talos, gam), talos.ptr(inv), rows, dim, talos.ptr(dx), talos.ptr(dg), 0)
        cs = torch.empty(dim, device="cuda:0"); talos.lib.talos_colsum(ctx.handle, dptr(talos, G), talos.ptr(cs), rows, dim, 0)
        ctx.synchronize(); outs.append((y, dx, dg, cs))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
