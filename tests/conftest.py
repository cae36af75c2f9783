import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for item in items:
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 GPUs"))
        elif "gpu" in item.keywords and n < 1:
            item.add_marker(pytest.mark.skip(reason="needs a GPU"))
