import os
import sys

import pytest

# Device tensors the harness and the test helpers allocate are padded with guard zones that are verified after
# every GPU test (ingot_b200.guarded_empty / check_guards).
os.environ.setdefault("INGOT_TEST_CANARY", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "inference-agent_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _guard_zones_intact(request):
    yield
    if "gpu" not in request.keywords:
        return
    try:
        import torch
        if not torch.cuda.is_available():
            return
        import ingot_b200 as ib
    except Exception:
        return
    torch.cuda.synchronize()
    assert ib.check_guards() == 0, "a kernel wrote outside a tensor the test handed to it"
