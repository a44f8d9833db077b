import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch
    has_gpu = torch.cuda.is_available()
    ngpu = torch.cuda.device_count() if has_gpu else 0
    for item in items:
        if "gpu" in item.keywords and not has_gpu:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(autouse=True)
def _device_error_check(request):
    """After every GPU test, fail if a kernel reported a bounded-wait timeout or a bad index."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from gllm_b200.ops import _native as nv
            torch.cuda.synchronize()
            code = nv.device_error()
            assert code == 0, f"device error word = {code} ({nv.ERROR_NAMES.get(code)})"
