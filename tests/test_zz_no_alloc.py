"""The allocation-free column sum (talos_colsum_noalloc) against the regular entry point.

Runs last on purpose: it is an addition beside the path, so a failure here must not hide the result of
any other test in a stop-at-first-failure run.  It has to pass both alone in a fresh process and after
the rest of the suite, and on two calls in a row, because every call reuses one fixed scratch array that
still holds the previous call's partial sums."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_colsum_noalloc_matches_colsum_on_consecutive_calls(talos):
    import torch
    assert torch.cuda.is_available()
    ctx = talos.torch_context(0)
    gen = torch.Generator(device="cuda").manual_seed(1234)
    # second shape is smaller in both directions, so stale partial sums of the first call sit right next
    # to (and beyond) the region the second call uses
    for i, (rows, n, acc) in enumerate([(70000, 256, 0), (777, 33, 1), (5, 1024, 0), (65536, 32, 1)]):
        g = torch.randn(rows, n, device="cuda", generator=gen)
        start = torch.randn(n, device="cuda", generator=gen)
        want = start.clone(); got = start.clone()
        talos.lib.talos_colsum(ctx.handle, talos.ptr(g), talos.ptr(want), rows, n, acc)
        ctx.synchronize()
        # Creating the context resolved the scratch array's address (and made the driver set the array aside), so not
        # even the first call may change the amount of free device memory.
        free_before = torch.cuda.mem_get_info(0)[0]
        talos.lib.talos_colsum_noalloc(ctx.handle, talos.ptr(g), talos.ptr(got), rows, n, acc)
        ctx.synchronize()
        assert torch.cuda.mem_get_info(0)[0] == free_before, "call %d changed the free device memory" % i
        ref = g.double().sum(0) + (start.double() if acc else 0)
        scale = float(ref.abs().max())
        assert float((got.double() - want.double()).abs().max()) <= 1e-5 * scale, (rows, n)
        assert float((got.double() - ref).abs().max()) <= 1e-5 * scale, (rows, n)
    with pytest.raises(talos.TalosError) as e:      # beyond the fixed scratch: refused, not truncated
        g = torch.zeros(4, 1025, device="cuda"); o = torch.zeros(1025, device="cuda")
        talos.lib.talos_colsum_noalloc(ctx.handle, talos.ptr(g), talos.ptr(o), 4, 1025, 0)
    assert e.value.status == talos.ERR_UNSUPPORTED and "1024 columns" in str(e.value)
    ctx.close()
