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
        B200Runtime.initialize_exclusive(RuntimeOptions(device=0))
    return B200Runtime.client(B200Runtime._device)
