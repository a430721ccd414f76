from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture
def cuda() -> torch.device:
    if not torch.cuda.is_available():
        pytest.skip("CUDA is not available")
    return torch.device("cuda")


def pytest_sessionfinish(session, exitstatus):
    import parity_bounds

    parity_bounds.write_report()


@pytest.fixture(autouse=True)
def device_status_stays_clear(request):
    """After every GPU test the library's device-side status word must still be zero: a bounded wait that gave up
    leaves its outputs undefined and makes later tensor kernels return at once until the word is cleared."""
    yield
    if request.node.get_closest_marker("gpu") is not None and torch.cuda.is_available():
        from oops_b200.runtime import cabi

        status = cabi.device_status(reset=True)
        assert status == 0, f"a kernel of this test recorded device status {status} ({cabi.status_message(status)})"


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """Build the C-ABI library once if it is stale (nvcc cross-compiles without a GPU)."""
    from oops_b200.csrc.build import build

    build()
