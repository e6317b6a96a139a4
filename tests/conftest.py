import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    if os.environ.get("VADE_TEST_POISON", "0") == "1":
        # every torch.empty() comes back filled with NaN / the largest integer: a kernel that reads memory it (or its
        # producer) never wrote, or that leaves part of its output unwritten, shows up as a failed comparison
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.utils.deterministic.fill_uninitialized_memory = True


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
