"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the headers
declare, and reports errors as status codes (no compute calls without a GPU)."""
import ctypes as C
import os

import pytest


def test_library_exports_every_declared_symbol(talos):
    protos = talos.parse_headers()
    assert len(protos) >= 38
    for name in protos:
        assert hasattr(talos.lib.cdll, name), "header declares %s but the library does not export it" % name


def test_header_parse_types(talos):
    protos = talos.parse_headers()
    res, args = protos["talos_gemm"]
    assert res is C.c_int32 and len(args) == 14
    assert args[0] is C.c_void_p and args[3] is C.c_int64 and args[12] is C.c_int32 and args[13] is C.c_void_p
    res, args = protos["talos_rmsnorm_fwd"]
    assert args[3] is C.c_float and args[4] is C.c_int64
    assert protos["talos_last_error_string"][0] is C.c_char_p
    assert protos["talos_ctx_launch_count"][0] is C.c_int64


def test_no_cpu_fallback_without_device(talos):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(talos.TalosError) as e:
        talos.Context(0)
    assert e.value.status == talos.ERR_CUDA and "no CPU path" in str(e.value)


def test_host_rng_matches_oracle_bit_for_bit(talos):
    import numpy as np
    import oracle as orc
    n = 4097
    out = np.empty(n, dtype=np.float32)
    talos.lib.talos_rng_normal_host(30, 0.0, 1.0, talos.ptr(out), n)
    assert np.array_equal(out, orc.rng_normal(30, (n,)).astype(np.float32))
    talos.lib.talos_rng_uniform_host(42, -1.0, 1.0, talos.ptr(out), n)
    assert np.array_equal(out, orc.rng_uniform(42, (n,), -1.0, 1.0).astype(np.float32))
    acts = np.empty(n, dtype=np.int32)
    talos.lib.talos_rng_bounded_host(31, 16, talos.ptr(acts), n)
    assert np.array_equal(acts, orc.rng_bounded(31, n, 16))
    d = np.empty(64, dtype=np.float64)
    talos.lib.talos_lcg_rand_host(42, -1.0, 1.0, talos.ptr(d), 64)
    assert np.array_equal(d, orc.lcg_rand((64,), -1.0, 1.0, 42))


def test_null_and_bad_arguments_are_status_codes(talos):
    with pytest.raises(talos.TalosError) as e:
        talos.lib.talos_rng_bounded_host(1, 0, None, 4)
    assert e.value.status == talos.ERR_ARG
    with pytest.raises(talos.TalosError):
        talos.lib.talos_ctx_synchronize(None)
    assert talos.lib.talos_ctx_launch_count(None) == 0
