import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "zendnn-pytorch-plugin_b200", ROOT / "oracle", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return dict(np.load(ROOT / "tests" / "golden" / "zentorch_golden.npz"))


@pytest.fixture(scope="session")
def c_oracle():
    from _util import load_c_oracle
    return load_c_oracle()


@pytest.fixture(scope="session")
def zt():
    """The package under test; importing it loads the native libraries or fails."""
    import zentorch_b200
    return zentorch_b200


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test, no kernel may have reported an expired device-side wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        from zentorch_b200 import _capi
        torch.cuda.synchronize()
        assert _capi.poll_device_status(reset=True) == 0, "a kernel reported a bounded-wait timeout"
