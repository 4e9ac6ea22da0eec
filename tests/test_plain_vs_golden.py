"""The plain implementation against harleyszhang/rapid_llm's own model code.

``tests/golden/tiny_{A,B}.npz`` hold logits the reference produced on the CPU in float32
for the tiny random models (see ``tests/golden/make_golden.py``); the folders are rebuilt
here from the same seeds.
"""

from pathlib import Path

import numpy as np
import pytest
import torch
from plain_qwen3 import forward_logits

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_logits(name, tiny_plain):
    config, weights = tiny_plain[name]
    data = np.load(GOLDEN / f"tiny_{name}.npz")
    index = 0
    while f"prompt{index}" in data:
        prompt = data[f"prompt{index}"].tolist()
        want = torch.from_numpy(data[f"logits{index}"])
        got = forward_logits(config, weights, prompt)
        assert got.shape == want.shape
        torch.testing.assert_close(got, want, rtol=1e-4, atol=2e-5)
        index += 1
    assert index >= 3


def test_plain_float64_agrees_with_float32(tiny_plain):
    config, weights = tiny_plain["C"]
    prompt = torch.randint(0, config["vocab_size"], (70,)).tolist()
    low = forward_logits(config, weights, prompt, torch.float32)
    high = forward_logits(config, weights, prompt, torch.float64)
    torch.testing.assert_close(low.double(), high, rtol=1e-4, atol=2e-5)


def test_window_changes_logits_only_past_the_window(tiny_plain):
    config, weights = tiny_plain["C"]
    prompt = torch.randint(0, config["vocab_size"], (90,)).tolist()
    windowed = forward_logits(config, weights, prompt)
    full_config = dict(config, use_sliding_window=False, layer_types=None)
    full = forward_logits(full_config, weights, prompt)
    window = config["sliding_window"]
    torch.testing.assert_close(windowed[:window], full[:window], rtol=1e-5, atol=1e-6)
    assert (windowed[window + 8 :] - full[window + 8 :]).abs().max() > 1e-4
