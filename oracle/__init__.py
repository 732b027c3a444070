"""CPU oracle for the Talos-XII dense neural path -- TEST INFRASTRUCTURE ONLY.

ctypes bindings to ``liboracle.so`` (the plain-C f64 restatement in ``talos_oracle.c``; each
C function cites the reference file:line it follows) plus numpy conveniences.  Only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this
package; the shipped library never does.

Parity status: scalar primitives, matmul forward/backward, broadcast and transpose are
pinned by the reference crate's own known-answer tests; the values of RMSNorm, RoPE,
softmax, batched matmul, MLA, PPO loss and Adam are "parity unpinned" (no reference test
fixes a number) and are validated by finite differences and cross-path checks instead.
"""
import ctypes as C
import os
import subprocess

import math
import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force=False):
    """Compile liboracle.so with the Makefile next to this file."""
    src = os.path.join(_HERE, "talos_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    if not os.path.exists(_LIB_PATH):
        build()
    return C.CDLL(_LIB_PATH)


_lib = _load()
_dp = C.POINTER(C.c_double)
_lp = C.POINTER(C.c_long)


def _p(a):
    return a.ctypes.data_as(_dp)


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def default_threads():
    """available_parallelism - 1, the reference's worker_reserve_cores = 1 default
    (src/worker.rs:60-67, src/config.rs:467)."""
    return max(1, (os.cpu_count() or 2) - 1)


_lib.orc_dot_product.restype = C.c_double
_lib.orc_softmax_exp_sum.restype = C.c_double
_lib.orc_sum_f64.restype = C.c_double
_lib.orc_sum_sq_diff.restype = C.c_double

# ---------------------------------------------------------------- simd.rs


def add_scaled_row(out, row, scale):
    out = _f64(out).copy(); row = _f64(row)
    _lib.orc_add_scaled_row(_p(out), _p(row), C.c_double(scale), C.c_long(out.size))
    return out


def dot_product(a, b):
    a = _f64(a); b = _f64(b)
    return _lib.orc_dot_product(_p(a), _p(b), C.c_long(a.size))


def vector_fma(dst, a, b):
    dst = _f64(dst).copy(); a = _f64(a); b = _f64(b)
    _lib.orc_vector_fma(_p(dst), _p(a), _p(b), C.c_long(dst.size))
    return dst


def vector_scale(row, s):
    row = _f64(row).copy()
    _lib.orc_vector_scale(_p(row), C.c_double(s), C.c_long(row.size))
    return row


def softmax_exp_sum(row):
    row = _f64(row).copy()
    s = _lib.orc_softmax_exp_sum(_p(row), C.c_long(row.size))
    return row, s


def sum_f64(v):
    v = _f64(v); return _lib.orc_sum_f64(_p(v), C.c_long(v.size))


def sum_sq_diff(v, mean):
    v = _f64(v); return _lib.orc_sum_sq_diff(_p(v), C.c_double(mean), C.c_long(v.size))


def normalize_slice(v, mean, std):
    v = _f64(v); out = np.empty_like(v)
    _lib.orc_normalize_slice(_p(v), _p(out), C.c_double(mean), C.c_double(std), C.c_long(v.size))
    return out


def gae(rewards, values, terminals, rew_mean, rew_var, gamma=0.99, lam=0.95):
    """Reward normalisation + reverse GAE scan (src/ppo.rs:650-671; GAMMA, GAE_LAMBDA at :18-19).  Returns
    (advantages, returns)."""
    r = _f64(rewards); v = _f64(values); t = np.ascontiguousarray(terminals, dtype=np.int32)
    adv = np.empty_like(r); ret = np.empty_like(r)
    _lib.orc_gae(_p(r), _p(v), t.ctypes.data_as(C.POINTER(C.c_int32)), C.c_long(r.size), C.c_double(gamma), C.c_double(lam),
                 C.c_double(rew_mean), C.c_double(rew_var), _p(adv), _p(ret))
    return adv, ret


class RunningMeanStd:
    """src/ppo.rs:444-480: count starts at 1e-4, mean 0, var 1; update() folds in one reward at a time."""

    def __init__(self):
        self.count, self.mean, self.var = C.c_double(1e-4), C.c_double(0.0), C.c_double(1.0)

    def update(self, xs):
        x = _f64(np.atleast_1d(xs))
        _lib.orc_running_mean_std_update(C.byref(self.count), C.byref(self.mean), C.byref(self.var), _p(x), C.c_long(x.size))

    def normalize(self, x):
        return (x - self.mean.value) / (math.sqrt(self.var.value) + 1e-8)

# ---------------------------------------------------------------- autograd.rs


def lcg_rand(shape, lo, hi, seed):
    """Tensor::rand (src/autograd.rs:114-124)."""
    out = np.empty(int(np.prod(shape)), dtype=np.float64)
    _lib.orc_lcg_rand(_p(out), C.c_long(out.size), C.c_double(lo), C.c_double(hi), C.c_uint64(seed))
    return out.reshape(shape)


def matmul(A, B, threads=None):
    A = _f64(A); B = _f64(B)
    A2 = A.reshape(1, -1) if A.ndim == 1 else A
    M, K = A2.shape; K2, N = B.shape
    assert K == K2, "MatMul dimension mismatch"
    Cm = np.empty((M, N), dtype=np.float64)
    _lib.orc_matmul_fwd(_p(A2), _p(B), _p(Cm), C.c_long(M), C.c_long(K), C.c_long(N),
                        C.c_int(threads or default_threads()))
    return Cm.reshape(N) if A.ndim == 1 else Cm


def matmul_bwd(A, B, G, dA=None, dB=None, threads=None, need_dA=True, need_dB=True):
    """Accumulates G.B^T into dA and A^T.G into dB (zeros if not given)."""
    A = _f64(A).reshape(-1, B.shape[0]); B = _f64(B); G = _f64(G).reshape(A.shape[0], B.shape[1])
    M, K = A.shape; N = B.shape[1]
    if need_dA and dA is None: dA = np.zeros((M, K))
    if need_dB and dB is None: dB = np.zeros((K, N))
    _lib.orc_matmul_bwd(_p(A), _p(B), _p(G), _p(dA) if need_dA else None, _p(dB) if need_dB else None,
                        C.c_long(M), C.c_long(K), C.c_long(N), C.c_int(threads or default_threads()))
    return dA, dB


def bias_add(Y, b):
    Y = _f64(Y).copy(); b = _f64(b)
    _lib.orc_bias_add(_p(Y), _p(b), C.c_long(Y.size // b.size), C.c_long(b.size))
    return Y


def bias_bwd(G, n_out):
    G = _f64(G); db = np.zeros(n_out)
    _lib.orc_bias_bwd(_p(G), _p(db), C.c_long(G.size // n_out), C.c_long(n_out))
    return db


def transpose(x, d0, d1, backward=False):
    """Tensor::transpose (src/autograd.rs:632-739).  With backward=True `x` is a gradient in
    the transposed layout and the result is the gradient scattered to the original layout."""
    x = _f64(x)
    if backward:
        orig = list(x.shape); orig[d0], orig[d1] = orig[d1], orig[d0]
        shape = (C.c_long * x.ndim)(*orig); out = np.zeros(orig)
    else:
        new = list(x.shape); new[d0], new[d1] = new[d1], new[d0]
        shape = (C.c_long * x.ndim)(*x.shape); out = np.empty(new)
    _lib.orc_transpose(_p(x), _p(out), shape, C.c_int(x.ndim), C.c_int(d0), C.c_int(d1), C.c_int(int(backward)))
    return out

# ---------------------------------------------------------------- nn.rs


def rmsnorm_fwd(x, w, eps):
    x = _f64(x); w = _f64(w); dim = w.size; rows = x.size // dim
    y = np.empty_like(x); rms = np.empty(rows); xhat = np.empty_like(x)
    _lib.orc_rmsnorm_fwd(_p(x), _p(w), C.c_double(eps), C.c_long(rows), C.c_long(dim), _p(y), _p(rms), _p(xhat))
    return y, rms, xhat


def rmsnorm_bwd(g, w, rms, xhat):
    g = _f64(g); w = _f64(w); dim = w.size; rows = g.size // dim
    dx = np.zeros_like(g); dw = np.zeros(dim)
    _lib.orc_rmsnorm_bwd(_p(g), _p(w), _p(_f64(rms)), _p(_f64(xhat)), C.c_long(rows), C.c_long(dim), _p(dx), _p(dw))
    return dx, dw


def linear_forward_inference(x, W, b=None):
    x = _f64(x); W = _f64(W); in_dim, out_dim = W.shape; rows = x.size // in_dim
    out = np.empty(rows * out_dim)
    bb = _f64(b) if b is not None else None
    _lib.orc_linear_forward_inference(_p(x), _p(W), _p(bb) if bb is not None else None, C.c_long(rows),
                                      C.c_long(in_dim), C.c_long(out_dim), _p(out))
    return out

# ---------------------------------------------------------------- transformer.rs


def rope_table(dim, max_len, base=10000.0):
    cosv = np.empty(max_len * (dim // 2)); sinv = np.empty_like(cosv)
    _lib.orc_rope_table(C.c_long(dim), C.c_long(max_len), C.c_double(base), _p(cosv), _p(sinv))
    return cosv, sinv


def rope(x, cosv, sinv, start_pos=0, backward=False):
    """RoPE::forward / its backward: rotates by the index along x.shape[-2] (src/transformer.rs:262)."""
    x = _f64(x); dim = x.shape[-1]; seq = x.shape[-2]; batches = x.size // (seq * dim)
    out = np.zeros_like(x) if backward else np.empty_like(x)
    _lib.orc_rope(_p(x), _p(out), _p(cosv), _p(sinv), C.c_long(batches), C.c_long(seq), C.c_long(dim),
                  C.c_long(start_pos), C.c_int(int(backward)))
    return out


def rope_token(x, cosv, sinv, start_pos=0):
    """Token-position rotation of [B,S,H,dr] (inference convention, src/transformer.rs:583-610)."""
    x = _f64(x); B, S, H, dr = x.shape; out = np.empty_like(x)
    _lib.orc_rope_token(_p(x), _p(out), _p(cosv), _p(sinv), C.c_long(cosv.size), C.c_long(B), C.c_long(S),
                        C.c_long(H), C.c_long(dr), C.c_long(start_pos))
    return out


def bmm_qkt(q, k, threads=None):
    q = _f64(q); k = _f64(k); B, S, D = q.shape; out = np.empty((B, S, S))
    _lib.orc_bmm_qkt_fwd(_p(q), _p(k), _p(out), C.c_long(B), C.c_long(S), C.c_long(D), C.c_int(threads or default_threads()))
    return out


def bmm_qkt_bwd(q, k, g, threads=None):
    q = _f64(q); k = _f64(k); g = _f64(g); B, S, D = q.shape
    dq = np.zeros_like(q); dk = np.zeros_like(k)
    _lib.orc_bmm_qkt_bwd(_p(q), _p(k), _p(g), _p(dq), _p(dk), C.c_long(B), C.c_long(S), C.c_long(D),
                         C.c_int(threads or default_threads()))
    return dq, dk


def bmm_pv(p, v, threads=None):
    p = _f64(p); v = _f64(v); B, S, Dv = v.shape; out = np.empty((B, S, Dv))
    _lib.orc_bmm_pv_fwd(_p(p), _p(v), _p(out), C.c_long(B), C.c_long(S), C.c_long(Dv), C.c_int(threads or default_threads()))
    return out


def bmm_pv_bwd(p, v, g, threads=None):
    p = _f64(p); v = _f64(v); g = _f64(g); B, S, Dv = v.shape
    dp = np.zeros_like(p); dv = np.zeros_like(v)
    _lib.orc_bmm_pv_bwd(_p(p), _p(v), _p(g), _p(dp), _p(dv), C.c_long(B), C.c_long(S), C.c_long(Dv),
                        C.c_int(threads or default_threads()))
    return dp, dv


def softmax(x, causal_period=0):
    x = _f64(x); n = x.shape[-1]; y = np.empty_like(x)
    _lib.orc_softmax_fwd(_p(x), _p(y), C.c_long(x.size // n), C.c_long(n), C.c_long(causal_period))
    return y


def softmax_bwd(y, g):
    y = _f64(y); g = _f64(g); n = y.shape[-1]; dx = np.zeros_like(y)
    _lib.orc_softmax_bwd(_p(y), _p(g), _p(dx), C.c_long(y.size // n), C.c_long(n))
    return dx

# ---------------------------------------------------------------- rng.rs


def rng_u64(seed, n):
    out = np.empty(n, dtype=np.uint64)
    _lib.orc_rng_u64(C.c_uint64(seed), out.ctypes.data_as(C.POINTER(C.c_uint64)), C.c_long(n))
    return out


def rng_uniform(seed, shape, lo=0.0, hi=1.0):
    out = np.empty(int(np.prod(shape)))
    _lib.orc_rng_uniform(C.c_uint64(seed), C.c_double(lo), C.c_double(hi), _p(out), C.c_long(out.size))
    return out.reshape(shape)


def rng_normal(seed, shape, mean=0.0, std=1.0):
    out = np.empty(int(np.prod(shape)))
    _lib.orc_rng_normal(C.c_uint64(seed), C.c_double(mean), C.c_double(std), _p(out), C.c_long(out.size))
    return out.reshape(shape)


def rng_bounded(seed, n, rng_range):
    out = np.empty(n, dtype=np.int32)
    _lib.orc_rng_bounded(C.c_uint64(seed), C.c_uint64(rng_range), out.ctypes.data_as(C.POINTER(C.c_int32)), C.c_long(n))
    return out


def f32r(a):
    """Round to fp32 and return as f64: the value both the oracle and the GPU consume."""
    return np.asarray(a, dtype=np.float32).astype(np.float64)
