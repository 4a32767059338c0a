import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")
    config.addinivalue_line("markers", "launches_allowed: a CPU test that runs outside validate-only mode")


@pytest.fixture(scope="session", autouse=True)
def _library_built():
    """The C-ABI library is built in-tree (seconds when the sources have not changed: the build
    keeps a digest); the suite does not depend on someone having built it before."""
    from g4b_b200 import build

    build.build()


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _cpu_tests_never_launch(request):
    """Every test that is not a GPU test runs with the library in validate-only mode: argument
    checks run, nothing is launched, so no CPU test can hand a host pointer to a kernel."""
    if request.node.get_closest_marker("gpu") is not None or request.node.get_closest_marker("launches_allowed") is not None:
        yield
        return
    from g4b_b200 import _cabi

    with _cabi.validate_only():
        yield


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test: no kernel may have recorded a failed bounded wait or a bad index."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch

    if torch.cuda.is_available():
        from g4b_b200 import _cabi

        status = _cabi.device_status()
        assert status == 0, f"device status word = {status:#x}"
