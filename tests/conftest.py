"""pytest configuration: the `gpu` marker and the import path of the repository root."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def gpu():
    """Device 0 of the CUDA library; a GPU test on a machine without a device is an error, not a skip."""
    import eidola_b200 as eb
    n = eb.device_count()
    if n == 0:
        pytest.fail("no CUDA device: GPU tests must run on the GPU box (select CPU tests with -m 'not gpu')")
    eb.capi.call("eb_device_set", eb.capi.c_i32(0))
    info = eb.device_info(0)
    yield info
    assert eb.status_read() == 0, "a kernel raised the device status word"
