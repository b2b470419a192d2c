import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs more than one CUDA device")


# GPU tests of these files were written after the last hardware run of the suite: they are collected after the files
# whose GPU tests have already passed on a B200, so that `-x` stopping at a failure among them cannot hide the rest.
_RUN_LAST = ("test_fp8.py", "test_lfm2.py", "test_gpt_oss.py", "test_expert_cache.py", "test_kv_residency.py",
             "test_weight_residency.py", "test_recurrent.py", "test_qwen_next.py")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        items.sort(key=lambda it: 1 if it.fspath.basename in _RUN_LAST else 0)   # stable: order inside a group is kept
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
