import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the native library")


@pytest.fixture(scope="session")
def native_ops():
    """Build (if needed) and load the native library; GPU tests depend on it so that they can
    never pass on a silent eager fallback."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from terracemoe_simulator_b200.ops import build as _build
    _build.build()
    from terracemoe_simulator_b200 import ops
    ops.reset()
    st = ops.status()
    assert st.loaded, st.reason
    return ops
