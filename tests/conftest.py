import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs several CUDA devices; skipped when fewer are visible")


def gpu_count():
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


@pytest.fixture(scope="session")
def native():
    from ep_xpress_b200 import native as loader
    return loader.load()
