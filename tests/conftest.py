import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "slow: long-running")


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


@pytest.fixture(scope="session")
def tiny_cfg():
    from oxibonsai_b200.core import Qwen3Config
    return Qwen3Config(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=1000, context=512, name="tiny")


@pytest.fixture(scope="session")
def tiny_gguf(tmp_path_factory, tiny_cfg):
    from oxibonsai_b200.core import write_synthetic_gguf
    p = tmp_path_factory.mktemp("gguf") / "tiny_tq2.gguf"
    write_synthetic_gguf(str(p), tiny_cfg, seed=42)
    return str(p)


@pytest.fixture(scope="session")
def tiny_q1_gguf(tmp_path_factory, tiny_cfg):
    from oxibonsai_b200.core import write_synthetic_gguf, Q1_0_G128
    p = tmp_path_factory.mktemp("gguf") / "tiny_q1.gguf"
    write_synthetic_gguf(str(p), tiny_cfg, weight_type=Q1_0_G128, tied=False, seed=7)
    return str(p)
