"""Configurations drawn at random (by seed, so every run draws the same) against the plain implementation.

The tiny configurations A, B and C are three points; the kernels promise every size the configuration
allows.  Each draw here varies all of them at once: head sizes of 16 to 256, groups of 1 to 7 query heads a
key/value head, widths, intermediate sizes and vocabularies that are multiples of 8 or not (the tensor-core
product or the library's), one to four layers, windows on some layers, tied or untied heads, pages of 8 to 32
tokens.  A draw replays a mixed trace (portions of prompts beside decoded tokens, so few pages that they are
used again) in bfloat16 and in float32, and decodes its last tokens from captured graphs.
"""

from __future__ import annotations

import random

import pytest
import torch
from plain_qwen3 import forward_logits, load_model_dir
from tolerances import for_dtype
from trace_tools import collect, mixed

DRAWS = 16
# by seed: small and large sizes, steps of 16 between them, the tensor-core kernels' size most often
HEAD_DIMS = [128, 16, 64, 128, 48, 32, 128, 96, 80, 128, 112, 256, 144, 128, 192, 64]


def draw_config(seed: int) -> tuple[dict, int]:
    rng = random.Random(1000 + seed)
    head_dim = HEAD_DIMS[seed % len(HEAD_DIMS)]
    kv_heads = rng.choice([1, 2, 3, 4])
    group = rng.choice([1, 2, 3, 4, 5, 7])
    while kv_heads * group > 14:
        kv_heads -= 1
    layers = rng.randint(1, 4)
    window = rng.choice([None, None, rng.randint(20, 70)])
    raw = {
        "architectures": ["Qwen3ForCausalLM"],
        "model_type": "qwen3",
        "vocab_size": rng.randint(90, 700),
        "hidden_size": rng.choice([40, 72, 100, 136, 200]),
        "intermediate_size": rng.choice([48, 88, 130, 176, 264]),
        "num_hidden_layers": layers,
        "num_attention_heads": kv_heads * group,
        "num_key_value_heads": kv_heads,
        "head_dim": head_dim,
        "max_position_embeddings": 256,
        "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6]),
        "rope_theta": rng.choice([1.0e4, 5.0e4, 1.0e6]),
        "tie_word_embeddings": rng.random() < 0.5,
        "attention_bias": False,
        "hidden_act": "silu",
        "sliding_window": window,
        "use_sliding_window": window is not None,
        "torch_dtype": "float32",
    }
    if window is not None:
        kinds = [rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)]
        kinds[rng.randrange(layers)] = "sliding_attention"
        raw["layer_types"] = kinds
        raw["max_window_layers"] = 0
    return raw, rng.choice([8, 16, 32])


def test_the_draws_differ():
    """The sweep is worth its time only if the draws spread over the options."""
    drawn = [draw_config(seed)[0] for seed in range(DRAWS)]
    assert len({raw["head_dim"] for raw in drawn}) >= 3
    assert len({raw["num_attention_heads"] // raw["num_key_value_heads"] for raw in drawn}) >= 3
    assert any(raw["sliding_window"] for raw in drawn) and any(raw["sliding_window"] is None for raw in drawn)
    assert any(raw["hidden_size"] % 8 for raw in drawn) or any(raw["intermediate_size"] % 8 for raw in drawn)


def _compare(rows, plain, dtype, label):
    tolerance = for_dtype(dtype)
    for request_id, by_position in rows.items():
        for position, got in sorted(by_position.items()):
            try:
                torch.testing.assert_close(got, plain[request_id][position], **tolerance)
            except AssertionError as exc:
                raise AssertionError(f"{label}: request {request_id!r}, position {position}: {exc}") from None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(DRAWS))
def test_a_drawn_configuration_mixed_and_decoding_from_graphs(seed, dtype, tmp_path):
    from rapid_llm_b200.config import EngineConfig, Qwen3Config, parse_dtype
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.replay import Replayer, engine_config_for
    from rapid_llm_b200.weights import write_random_model

    raw, page = draw_config(seed)
    label = f"seed {seed}: {raw}, page {page}"
    torch_dtype = parse_dtype(dtype)
    folder = write_random_model(tmp_path / "model", Qwen3Config.from_dict(raw), 50 + seed, dtype=torch_dtype)
    config, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(seed)
    lengths = [37, 120, 18, 75, 201, 52]
    sequences = {f"r{index}": torch.randint(0, raw["vocab_size"], (length,), generator=generator).tolist()
                 for index, length in enumerate(lengths)}
    plain = {rid: forward_logits(config, weights, tokens) for rid, tokens in sequences.items()}

    # portions of some beside decoded tokens of others, with so few pages that they are used again
    records, peak = mixed(sequences, seed=seed, max_live=3, page=page)
    model_config = Qwen3Config.from_dict(raw)
    runner = ModelRunner.from_folder(folder, engine_config_for(model_config, dtype, peak, page, 3))
    replayer, outputs = Replayer(runner), {}
    for record in records:
        out = replayer.run_step(record)
        if out is not None:
            outputs[record["step"]] = torch.from_numpy(out.copy())
        runner.cache.check()
    _compare(collect(records, outputs), plain, dtype, label + " (mixed)")
    del runner, replayer

    # two requests whole but for their tails, the tails decoded together from captured graphs
    names = ["r1", "r4"]
    engine = EngineConfig(dtype=torch_dtype, max_seq_len=256, page_size=page, num_pages=2 * (-(-256 // page)) + 1,
                          max_num_seqs=3, max_num_batched_tokens=256, max_chunk_size=256, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    tail = 12
    for name in names:
        assert runner.admit(name)
        tokens = sequences[name]
        logits = runner.step([StepEntry(name, tokens[:-tail], [len(tokens) - tail - 1])])
        _compare({name: {len(tokens) - tail - 1: logits[0].float().cpu()}}, plain, dtype, label + " (prompt)")
    for offset in range(tail):
        entries = [StepEntry(name, [sequences[name][len(sequences[name]) - tail + offset]], [0]) for name in names]
        logits = runner.step_decode(entries).float().cpu()
        for row, name in enumerate(names):
            position = len(sequences[name]) - tail + offset
            _compare({name: {position: logits[row]}}, plain, dtype, label + " (graph decode)")
    for name in names:
        runner.release(name)
    runner.check_fault()
    runner.cache.check()
