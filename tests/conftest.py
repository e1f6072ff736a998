import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu(n): needs at least n CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch

    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for item in items:
        m = item.get_closest_marker("multigpu")
        if m is not None:
            need = int(m.args[0]) if m.args else 2
            if n < need:
                item.add_marker(pytest.mark.skip(reason=f"needs {need} GPUs, found {n}"))
        elif item.get_closest_marker("gpu") is not None and n == 0:
            item.add_marker(pytest.mark.skip(reason="needs a GPU"))
