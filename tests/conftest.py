import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (ROOT, os.path.join(ROOT, 'tests')):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc
    orc.build()
    return orc


@pytest.fixture(scope="session")
def client():
    """One process-wide runtime context, as the reference allows exactly one (runtime/mod.rs:424-435)."""
    from rust_ascend_b200 import B200Runtime, RuntimeOptions
    if B200Runtime._ctx is None:
        # every allocation of the GPU tests is surrounded by guard bands and starts as NaN patterns: an out-of-bounds store or an
        # output element a kernel forgot shows up (no memory checker can run on the GPU pool these tests use)
        os.environ.setdefault("RUDA_GUARD_BANDS", "1")
        B200Runtime.initialize_exclusive(RuntimeOptions(device=0))
    return B200Runtime.client(B200Runtime._device)


@pytest.fixture(autouse=True)
def _guard_bands_intact(request):
    """After every GPU test: no kernel wrote outside an allocation."""
    yield
    from rust_ascend_b200 import B200Runtime
    if request.node.get_closest_marker("gpu") is not None and B200Runtime._ctx is not None:
        client = B200Runtime.client(B200Runtime._device)
        assert client.check_guards() == 0, "a kernel wrote outside an allocation (guard band damaged)"
