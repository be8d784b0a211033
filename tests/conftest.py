import os
import sys
from pathlib import Path

import pytest

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (sm_100a)")
    config.addinivalue_line("markers", "multigpu: test needs more than one CUDA device")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
        ngpu = torch.cuda.device_count() if has_gpu else 0
    except Exception:
        has_gpu, ngpu = False, 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and not has_gpu:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(skip_multi)


@pytest.fixture(autouse=True)
def _check_kernel_status(request):
    """After every GPU test, the device status word must be clean (no bounded wait ran out)."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from ferrotorch_b200 import _lib
            st = _lib.read_status()
            assert st == 0, f"kernel status word = {st:#x}"
