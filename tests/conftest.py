import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "needs_tensor_cores: in modes 1 / 2 the test's products are large enough that the tcgen05 path must be active afterwards")


@pytest.fixture(scope="session")
def talos():
    """The product package (directory name is not an identifier, so it is loaded by path)."""
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(autouse=True)
def _no_silent_fp32_stand_in(request):
    """After every GPU test that used a context: the tensor-core self-check must not have failed (a failure makes the
    fp32 CUDA-core kernel serve the TF32 / 3xTF32 modes, which keeps results right and would keep the suite green), and
    a test parametrised with a tensor-core mode that launched products large enough to need them must have had them."""
    yield
    if request.node.get_closest_marker("gpu") is None or "ctx" not in request.fixturenames:
        return
    ctx = request.getfixturevalue("ctx")
    if not getattr(ctx, "handle", None):
        return
    state = ctx.tensor_cores_state
    assert state != -1, "tensor-core self-check failed on this context: TF32 / 3xTF32 modes are running on the fp32 kernel"
    mode = request.node.callspec.params.get("mode") if hasattr(request.node, "callspec") else None
    if mode in (1, 2) and request.node.get_closest_marker("needs_tensor_cores"):
        assert state == 1, "this test's products should have run on the tensor cores"
