"""Shared fixtures: markers, tiny model folders (made in temporary folders, never committed)."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
for path in (str(ROOT), str(ROOT / "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, float32 weights, keyed 'A', 'B', 'C'."""
    from tiny_configs import CONFIGS, SEEDS

    from rapid_llm_b200.config import Qwen3Config
    from rapid_llm_b200.weights import write_random_model

    root = tmp_path_factory.mktemp("tiny_models")
    return {
        name: write_random_model(root / name, Qwen3Config.from_dict(raw), SEEDS[name], dtype=torch.float32)
        for name, raw in CONFIGS.items()
    }


@pytest.fixture(scope="session")
def tiny_dirs_bf16(tmp_path_factory):
    """The same configurations and seeds with the matrices stored in bfloat16."""
    from tiny_configs import CONFIGS, SEEDS

    from rapid_llm_b200.config import Qwen3Config
    from rapid_llm_b200.weights import write_random_model

    root = tmp_path_factory.mktemp("tiny_models_bf16")
    return {
        name: write_random_model(root / name, Qwen3Config.from_dict(raw), SEEDS[name], dtype=torch.bfloat16)
        for name, raw in CONFIGS.items()
    }


@pytest.fixture(scope="session")
def tiny_plain_bf16(tiny_dirs_bf16):
    from plain_qwen3 import load_model_dir

    return {name: load_model_dir(folder) for name, folder in tiny_dirs_bf16.items()}


@pytest.fixture(scope="session")
def tiny_plain(tiny_dirs):
    """``name -> (config dict, weights)`` as the plain implementation reads the folders."""
    from plain_qwen3 import load_model_dir

    return {name: load_model_dir(folder) for name, folder in tiny_dirs.items()}
