"""Helpers for the GPU parity tests: seeded fp32-representable inputs, device transfer, error norms."""
import numpy as np

import oracle as orc

TOL = {0: 1e-5, 1: 1e-5, 2: 2e-3}     # north-star tolerances: fp32 / 3xTF32 <= 1e-5, TF32 <= 2e-3 (relative)


def dev(a, dtype=None):
    import torch
    a = np.ascontiguousarray(a)
    if dtype is None:
        dtype = torch.int32 if a.dtype.kind in "iu" else torch.float32
    return torch.tensor(a, dtype=dtype, device="cuda:0")


def host(t):
    return t.detach().double().cpu().numpy()


def rel_err(got, ref):
    got = host(got) if hasattr(got, "detach") else np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64).reshape(got.shape)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(got - ref) / den) if den > 0 else float(np.linalg.norm(got))


def max_err(got, ref):
    got = host(got) if hasattr(got, "detach") else np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64).reshape(got.shape)
    den = np.abs(ref).max()
    return float(np.abs(got - ref).max() / den) if den > 0 else float(np.abs(got).max())


def normal(seed, shape, std=1.0):
    return orc.f32r(orc.rng_normal(seed, shape, 0.0, std))


def uniform(seed, shape, lo=-1.0, hi=1.0):
    return orc.f32r(orc.rng_uniform(seed, shape, lo, hi))


def xavier(seed, fan_in, fan_out):
    lim = float(np.sqrt(6.0 / (fan_in + fan_out)))
    return uniform(seed, (fan_in, fan_out), -lim, lim)
