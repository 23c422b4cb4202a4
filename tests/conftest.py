import os
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on a B200 with the kernel library built)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA GPUs")
    config.addinivalue_line("markers", "distributed: spawns several processes (gloo on CPU)")


def pytest_collection_modifyitems(config, items):
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for item in items:
        if "gpu" in item.keywords and n < 1:
            item.add_marker(pytest.mark.skip(reason="no CUDA GPU"))
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA GPUs"))


@pytest.fixture
def tiny_cfg():
    from nanonemo_b200.models.config import ModelConfig

    return ModelConfig(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, vocab_size=512, max_seq_len=64)
