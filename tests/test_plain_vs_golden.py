"""The plain implementation against harleyszhang/rapid_llm's own model code.

``tests/golden/tiny_{A,B}.npz`` hold logits the reference produced on the CPU in float32
for the tiny random models (see ``tests/golden/make_golden.py``); the folders are rebuilt
here from the same seeds.  ``tests/golden/sampling.npz`` holds what the reference's sampler
code makes of rows of random logits (``tests/golden/make_sampling_golden.py``), and
``tests/golden/greedy.npz`` the token ids the reference's continuous-batching engine generated
greedily, prompt portions of 13 tokens beside decode steps (``tests/golden/make_greedy_golden.py``).
"""

from pathlib import Path

import numpy as np
import pytest
import torch
from plain_qwen3 import forward_logits, greedy_generate, nucleus, penalised, sample_token

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


def test_plain_sampler_pieces_match_the_reference():
    """The repetition penalty, the greedy pick and the set of tokens the nucleus keeps, row by row."""
    data = np.load(GOLDEN / "sampling.npz")
    rows = data["logits"].shape[0]
    assert rows >= 20
    for row in range(rows):
        logits = torch.from_numpy(data["logits"][row])
        generated = data["generated"][row, : data["generated_count"][row]].tolist()
        temperature, top_p, penalty = float(data["temperature"][row]), float(data["top_p"][row]), float(data["penalty"][row])
        values = penalised(logits, generated, penalty)
        torch.testing.assert_close(values, torch.from_numpy(data["penalised"][row]), rtol=0, atol=0)
        assert sample_token(logits, 0.0, penalty=penalty, generated=generated) == int(data["greedy"][row])
        scaled = values / temperature
        kept = nucleus(torch.exp(scaled - scaled.max()), top_p)
        want = torch.from_numpy(data["kept"][row])
        # a token whose mass-before lies within rounding of top_p may fall on either side
        assert int((kept != want).sum()) <= 1, (row, int(kept.sum()), int(want.sum()))
        # every draw of the plain sampler lands inside the reference's nucleus
        for counter in range(6):
            assert want[sample_token(logits, temperature, top_p, penalty, generated, seed=row, counter=counter)] or (kept != want).any()


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_greedy_tokens_match_the_references_engine(name, tiny_plain):
    config, weights = tiny_plain[name]
    data = np.load(GOLDEN / "greedy.npz")
    index = 0
    while f"{name}_prompt{index}" in data:
        want = data[f"{name}_tokens{index}"].tolist()
        assert greedy_generate(config, weights, data[f"{name}_prompt{index}"].tolist(), len(want)) == want
        index += 1
    assert index >= 3
