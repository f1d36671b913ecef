"""Test tiers: everything unmarked runs on a CPU-only machine; ``gpu`` needs one B200;
``multigpu`` needs two or more; ``slow`` is excluded from quick runs."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
        ngpu = torch.cuda.device_count() if have else 0
    except Exception:
        have, ngpu = False, 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and not have:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(skip_multi)


@pytest.fixture
def fp8_fp32_scales():
    """Runs a test with fp32 block scales (epilogue promotion) instead of the default UE8M0 mode."""
    from hartsyinference_b200 import config
    config.set_override("fp8_scales", "fp32")
    yield
    config.set_override("fp8_scales", None)
