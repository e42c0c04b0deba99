import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from orinfer_b200.ops import native
    native.init()          # raises when the kernel library is missing: no silent fallback
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _kernel_status(request):
    """After every GPU test, no bounded wait may have run out."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from orinfer_b200.ops import native
            status = native.read_status()
            native.clear_status()
            assert status == 0, f"kernel status word {status:#x}"
