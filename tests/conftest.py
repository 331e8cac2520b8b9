import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def _gpu_available() -> bool:
    try:
        from zigrad_b200 import abi
        return bool(abi.lib().zg_device_available())
    except Exception:
        return False


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def dev():
    """One CudaDevice for the whole session.  GPU tests must fail, not skip,
    when the library is missing on a machine that has a GPU."""
    from zigrad_b200.device import CudaDevice
    if not _gpu_available():
        pytest.skip("no CUDA device")
    d = CudaDevice(0)
    yield d
    d.deinit()


@pytest.fixture()
def gpu(dev):
    """Per-test view of the device: fails the test if the library's sticky
    status was set while it ran."""
    from zigrad_b200 import abi
    abi.lib().zg_clear_error()
    yield dev
    dev.sync()
    abi.check()
