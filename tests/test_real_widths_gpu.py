"""One layer at the widths of Qwen3-8B (hidden 4096, 32 query heads over 8 of size 128, intermediate
12288) with the real vocabulary of 151,936 rows, in float32 and in bfloat16, against the plain
implementation: whole, the last 32 tokens one by one, portions of changing size, mixed with pages
used again, and decoding from a captured graph.

The output head at this size is 1,187 tiles of 128 rows: more than the tensor-core product has
CTAs, so each walks several tiles (two accumulator buffers, flipping phases) -- a path that no
smaller vocabulary reaches.  The float32 engine is also compared with itself: rows of different
cuttings of the same sequences are equal bit for bit, since no float32 reduction order depends on
the batch.

The embeddings are tied so that the folder holds the large table once.
"""

from __future__ import annotations

import pytest
import torch
from plain_qwen3 import forward_hidden, head_logits, load_model_dir
from test_engine_gpu import make_runner, random_tokens, replay
from tolerances import assert_rows_close
from trace_tools import collect, mixed, portions, tail_one_by_one, whole

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
VOCAB = 151936

REAL_WIDTHS = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": VOCAB, "hidden_size": 4096,
    "intermediate_size": 12288, "num_hidden_layers": 1, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "attention_bias": False, "hidden_act": "silu", "sliding_window": None,
    "use_sliding_window": False, "torch_dtype": "bfloat16",
}
LENGTHS = {"w": 200, "r0": 90, "r1": 150, "r2": 40, "r3": 70}


def asked(length: int):
    """Every 13th position, the edges of the first pages and the last three: a row of logits is 600 KB."""
    return lambda p: p % 13 == 0 or p in (1, 15, 16, 17, 63, 64) or p >= length - 3


class Plain:
    """The plain implementation's residual streams of the test sequences; logits row by row on demand."""

    def __init__(self, folder):
        self.config, self.weights = load_model_dir(folder)
        self.tokens = {name: random_tokens(VOCAB, count, 300 + index) for index, (name, count) in enumerate(LENGTHS.items())}
        self.hidden = {name: forward_hidden(self.config, self.weights, ids) for name, ids in self.tokens.items()}

    def logits(self, name: str, positions: list[int]) -> torch.Tensor:
        return head_logits(self.config, self.weights, self.hidden[name][positions])


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    from rapid_llm_b200.config import Qwen3Config
    from rapid_llm_b200.weights import write_random_model

    folder = write_random_model(tmp_path_factory.mktemp("real_widths") / "model", Qwen3Config.from_dict(REAL_WIDTHS), 21,
                                dtype=torch.bfloat16)
    return folder, Plain(folder)


def compare(rows: dict, plain: Plain, dtype: str) -> None:
    for name, by_position in rows.items():
        positions = sorted(by_position)
        want = plain.logits(name, positions)
        got = torch.stack([by_position[p] for p in positions])
        try:
            assert_rows_close(got, want, dtype)
        except AssertionError as exc:
            raise AssertionError(f"request {name!r}, positions {positions}: {exc}") from None


def ways_of_cutting(plain: Plain) -> dict[str, list[dict]]:
    tokens = plain.tokens["w"]
    wanted = asked(len(tokens))
    return {
        "whole": whole("w", tokens, wanted=wanted),
        "tail": tail_one_by_one("w", tokens, 32, wanted=wanted),
        "portions": portions("w", tokens, [61, 2, 33, 5, 64, 3, 17], wanted=wanted),
    }


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_tail_and_portions_at_real_widths(dtype, real):
    folder, plain = real
    runner = make_runner(folder, dtype, max_tokens=256, page_size=16)
    results = {}
    for label, records in ways_of_cutting(plain).items():
        rows = collect(records, replay(runner, records))
        assert rows["w"], label
        compare(rows, plain, dtype)
        results[label] = rows["w"]
    if dtype == "float32":
        # the cuttings against each other: no float32 sum depends on the batch or on the cut
        for label in ("tail", "portions"):
            for position, row in results[label].items():
                if position in results["whole"]:
                    assert torch.equal(row, results["whole"][position]), (label, position)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_with_pages_used_again_at_real_widths(dtype, real):
    folder, plain = real
    sequences = {name: ids for name, ids in plain.tokens.items() if name != "w"}
    wanted = lambda p: p % 11 == 0 or p in (15, 16, 31, 32)      # noqa: E731
    records, peak = mixed(sequences, seed=5, max_live=3, page=16, wanted=wanted)
    runner = make_runner(folder, dtype, max_tokens=peak, page_size=16, max_live=3)
    rows = collect(records, replay(runner, records))
    assert set(rows) == set(sequences)
    compare(rows, plain, dtype)
    if dtype == "float32":
        # each request alone and whole gives the same bits as in the mixed batches
        alone = make_runner(folder, dtype, max_tokens=256, page_size=16)
        for name, ids in sequences.items():
            records = whole(name, ids, wanted=lambda p, name=name: p in rows[name])
            single = collect(records, replay(alone, records))[name]
            for position, row in single.items():
                assert torch.equal(row, rows[name][position]), (name, position)


def test_decoding_from_a_graph_at_real_widths(real):
    """Three requests decoded together from a captured graph (a bucket of four): every step's output head
    walks its 1,187 tiles, the products before it split their inner range over clusters."""
    from rapid_llm_b200.config import EngineConfig
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry

    folder, plain = real
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=256, page_size=16, num_pages=40, max_num_seqs=4,
                          max_num_batched_tokens=256, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    names = ["r0", "r1", "r3"]
    at = {}
    for name in names:
        runner.admit(name)
        at[name] = LENGTHS[name] - 6
        runner.step([StepEntry(name, plain.tokens[name][: at[name]], [])])
    for _ in range(6):
        got = runner.step_decode([StepEntry(name, plain.tokens[name][at[name] : at[name] + 1], [0]) for name in names])
        got = got.float().cpu()
        for index, name in enumerate(names):
            assert_rows_close(got[index : index + 1], plain.logits(name, [at[name]]), "bfloat16")
            at[name] += 1
    runner.check_fault()
    runner.cache.check()
