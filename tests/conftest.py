import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# The engine runs a warm-up request from its constructor; the tests count requests, steps and cache hits exactly, so
# they switch it off (worker processes inherit the variable). tests/test_engine_features.py covers the warm-up itself.
os.environ.setdefault("DISABLE_WARMUP", "1")
# log records of the tests go to standard error instead of log/ksana_llm.log
os.environ.setdefault("KLLM_LOG_FILE", "stderr")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
