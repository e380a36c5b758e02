"""Shared pytest configuration.

Tests that need a GPU are marked ``gpu`` and are skipped on machines without a
CUDA device; everything else runs on CPU (multi-process cases use gloo over
127.0.0.1).
"""

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch

    has_cuda = torch.cuda.is_available()
    count = torch.cuda.device_count() if has_cuda else 0
    for item in items:
        if "gpu" in item.keywords and not has_cuda:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and count < 2:
            item.add_marker(pytest.mark.skip(reason="needs two CUDA devices"))


@pytest.fixture
def tiny_config():
    from systems_for_llms_b200.config import DataConfig, ModelConfig, TrainConfig

    return TrainConfig(model=ModelConfig(vocab_size=32, context_length=8, d_model=16, num_layers=2,
                                         num_heads=4, d_ff=32, attention_backend="sdpa"),
                       data=DataConfig(kind="synthetic", synthetic_tokens=256), seed=1337,
                       batch_size=2, max_steps=4, learning_rate=1e-3, min_learning_rate=1e-4,
                       warmup_steps=1, grad_clip=0.15, eval_interval=4, eval_batches=4,
                       eval_batch_size=1, checkpoint_interval=2)
