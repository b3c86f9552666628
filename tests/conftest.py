import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


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


def pytest_sessionfinish(session, exitstatus):
    """In-process tests may leave a default process group behind; tear it down (bounded) so the interpreter exits cleanly."""
    try:
        import threading

        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            return
        th = threading.Thread(target=dist.destroy_process_group, daemon=True)
        th.start()
        th.join(timeout=10.0)
    except Exception:
        pass
