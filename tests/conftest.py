"""Test configuration: markers are probes — a machine that lacks something skips, never fails."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multigpu(n): needs n CUDA devices")
    config.addinivalue_line("markers", "slow: long-running")


def _gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_collection_modifyitems(config, items):
    n = _gpu_count()
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        m = item.get_closest_marker("multigpu")
        if m is not None and n < int(m.args[0] if m.args else 2):
            item.add_marker(pytest.mark.skip(reason=f"needs {m.args[0] if m.args else 2} CUDA devices"))


@pytest.fixture(autouse=True)
def _clear_view_cache():
    yield
    try:
        from dataflow_b200.runtime.interop import invalidate_views
        invalidate_views()
    except Exception:
        pass
