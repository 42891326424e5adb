import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
        ngpu = torch.cuda.device_count() if have else 0
    except Exception:
        have, ngpu = False, 0
    for it in items:
        if "gpu" in it.keywords and not have:
            it.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in it.keywords and ngpu < 2:
            it.add_marker(pytest.mark.skip(reason="needs >= 2 GPUs"))
