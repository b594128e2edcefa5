import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _gpu_available() -> bool:
    if os.environ.get("B200OPS_FORCE_NO_GPU"):
        return False
    try:
        from compiler_b200.runtime import abi
        import ctypes
        props = abi.DeviceProps()
        return abi.lib().b200_device_query(0, ctypes.byref(props)) == 0
    except Exception:  # noqa: BLE001
        return False


@pytest.fixture(scope="session")
def device():
    """One B200Device for the whole session (GPU tests only)."""
    if not _gpu_available():
        pytest.skip("no CUDA device")
    from compiler_b200.device import B200Device
    return B200Device(0)
