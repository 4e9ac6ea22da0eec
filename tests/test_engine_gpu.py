"""The engine against the plain implementation, in float32 and in bfloat16.

Every test replays token ids through the step function (the loop behind ``bin/trace_run``)
and compares each wanted logits row with the plain implementation's row for the same
request and position: whole; most in one step and the last 32 one by one; portions of
changing size down to two tokens; mixed, up to four live requests with so few pages that
they are used again.
"""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
from plain_qwen3 import forward_logits
from tiny_configs import PAGE_SIZES
from tolerances import for_dtype
from trace_tools import collect, mixed, portions, tail_one_by_one, whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DTYPES = ["float32", "bfloat16"]


def make_runner(folder, dtype: str, max_tokens: int, page_size: int, max_live: int = 8):
    from rapid_llm_b200.config import load_config
    from rapid_llm_b200.engine.runner import ModelRunner
    from rapid_llm_b200.replay import engine_config_for

    config = load_config(folder)
    return ModelRunner.from_folder(folder, engine_config_for(config, dtype, max_tokens, page_size, max_live))


def replay(runner, records):
    from rapid_llm_b200.replay import Replayer

    replayer = Replayer(runner)
    outputs = {}
    for record in records:
        out = replayer.run_step(record)
        if out is not None:
            outputs[record["step"]] = torch.from_numpy(out.copy())
    runner.cache.check()
    return outputs


def random_tokens(vocab: int, count: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()


def compare(rows, plain_by_request, dtype):
    tolerance = for_dtype(dtype)
    for request_id, by_position in rows.items():
        want = plain_by_request[request_id]
        for position, got in sorted(by_position.items()):
            try:
                torch.testing.assert_close(got, want[position], **tolerance)
            except AssertionError as exc:
                raise AssertionError(f"request {request_id!r}, position {position}: {exc}") from None


@pytest.fixture(scope="module")
def models(tiny_dirs, tiny_dirs_bf16, tiny_plain, tiny_plain_bf16):
    return {
        "float32": (tiny_dirs, tiny_plain),
        "bfloat16": (tiny_dirs_bf16, tiny_plain_bf16),
    }


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_tail_and_portions(name, dtype, models):
    dirs, plains = models[dtype]
    config, weights = plains[name]
    limit = config["max_position_embeddings"]
    lengths = [5, 17, 33, min(100, limit - 1), min(limit - 1, 200)]
    runner = make_runner(dirs[name], dtype, max_tokens=limit, page_size=PAGE_SIZES[name])
    for index, length in enumerate(lengths):
        tokens = random_tokens(config["vocab_size"], length, 100 + index)
        plain = forward_logits(config, weights, tokens)
        cases = {
            "whole": whole("w", tokens),
            "tail": tail_one_by_one("t", tokens, 32),
            "portions": portions("p", tokens, [13, 2, 7, 31, 3, 2, 16, 5]),
        }
        for label, records in cases.items():
            rows = collect(records, replay(runner, records))
            request_id = records[0]["entries"][0]["id"]
            assert sorted(rows[request_id]) == list(range(length)), label
            compare(rows, {request_id: plain}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_with_pages_used_again(name, dtype, models, tmp_path):
    dirs, plains = models[dtype]
    config, weights = plains[name]
    limit = config["max_position_embeddings"]
    page = PAGE_SIZES[name]
    lengths = [40, 97, 23, 64, 120, 35, 77, 50, 18, 90]
    sequences = {
        f"r{index}": random_tokens(config["vocab_size"], min(length, limit - 1), 200 + index)
        for index, length in enumerate(lengths)
    }
    records, peak = mixed(sequences, seed=7, max_live=4, page=page)
    runner = make_runner(dirs[name], dtype, max_tokens=peak, page_size=page, max_live=4)
    from rapid_llm_b200.replay import Replayer

    replayer, outputs = Replayer(runner, tmp_path), {}
    for record in records:
        out = replayer.run_step(record)
        if out is not None:
            outputs[record["step"]] = torch.from_numpy(out.copy())
        runner.cache.check()
    # which request held which page, read from the files the replay wrote beside the logits
    owners: dict[tuple[int, int], set[str]] = {}
    for record in records:
        held = json.loads((tmp_path / f"{record['step']}.pages.json").read_text())
        assert set(held) == {entry["id"] for entry in record["entries"]}
        for request_id, groups in held.items():
            for group, pages in enumerate(groups):
                for page_id in pages:
                    if page_id:
                        owners.setdefault((group, page_id), set()).add(request_id)
    assert any(len(requests) > 1 for requests in owners.values()), "no page was used again"
    plain = {rid: forward_logits(config, weights, tokens) for rid, tokens in sequences.items()}
    compare(collect(records, outputs), plain, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype, models):
    """Positions 0, 1, 2 alone: a one-token prompt, then single tokens."""
    dirs, plains = models[dtype]
    config, weights = plains["B"]
    tokens = random_tokens(config["vocab_size"], 4, 5)
    runner = make_runner(dirs["B"], dtype, max_tokens=64, page_size=PAGE_SIZES["B"])
    records = tail_one_by_one("f", tokens, tail=3)
    rows = collect(records, replay(runner, records))
    compare(rows, {"f": forward_logits(config, weights, tokens)}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, models):
    """A short prompt followed by 200 single-token steps, past several page edges and the window."""
    dirs, plains = models[dtype]
    config, weights = plains["C"]
    tokens = random_tokens(config["vocab_size"], 230, 9)
    runner = make_runner(dirs["C"], dtype, max_tokens=256, page_size=PAGE_SIZES["C"])
    records = tail_one_by_one("d", tokens, tail=200)
    rows = collect(records, replay(runner, records))
    compare(rows, {"d": forward_logits(config, weights, tokens)}, dtype)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_norms_ride_on_the_products_of_small_steps(name, models, monkeypatch):
    """In bfloat16 steps of up to 64 tokens only the first and the last norm run as kernels; the
    others are taken along by the products around them.  Both ways give the plain implementation's
    logits, and larger steps keep the norm kernels."""
    from rapid_llm_b200.ops import gemm, kernels

    dirs, plains = models["bfloat16"]
    config, weights = plains[name]
    layers = config["num_hidden_layers"]
    tokens = random_tokens(config["vocab_size"], 90, 77)
    plain = forward_logits(config, weights, tokens)
    calls = []
    real = kernels.add_rmsnorm
    monkeypatch.setattr(kernels, "add_rmsnorm", lambda *a, **k: (calls.append(a[0].shape[0]), real(*a, **k))[1])
    results = {}
    for fused in (True, False):
        monkeypatch.setattr(gemm, "FUSE_NORMS", fused)
        runner = make_runner(dirs[name], "bfloat16", max_tokens=128, page_size=PAGE_SIZES[name])
        records = portions("n", tokens, [70, 9, 1, 1, 2, 7])      # a large step, then small ones
        calls.clear()
        outputs = replay(runner, records)
        per_step = 2 * layers + 1
        large = [rows for rows in calls if rows > 64]
        assert len(large) == per_step - 1 or len(large) == per_step    # the last norm sees the wanted rows only
        small_steps = len(records) - 1
        small = len(calls) - per_step
        assert small == (2 if fused else per_step) * small_steps, (fused, calls)
        rows = collect(records, outputs)
        compare(rows, {"n": plain}, "bfloat16")
        results[fused] = rows["n"]
    tolerance = for_dtype("bfloat16")
    for position, got in results[True].items():
        torch.testing.assert_close(got, results[False][position], **tolerance)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_products_of_small_steps_as_one_persistent_kernel(name, models, monkeypatch):
    """With ``ops.gemm.CHAIN`` the products that follow one another in a small bfloat16 step (output projection,
    gate/up, down, the next layer's q/k/v) are queued and run as one kernel; the logits are the plain
    implementation's, in portions and from a captured decode graph."""
    from rapid_llm_b200.engine.runner import StepEntry
    from rapid_llm_b200.ops import gemm, kernels

    dirs, plains = models["bfloat16"]
    config, weights = plains[name]
    tokens = random_tokens(config["vocab_size"], 90, 78)
    plain = forward_logits(config, weights, tokens)
    calls = []
    real = kernels.gemm_chain
    monkeypatch.setattr(kernels, "gemm_chain", lambda products, fault, **k: (calls.append(len(products)), real(products, fault, **k))[1])
    monkeypatch.setattr(gemm, "CHAIN", True)
    runner = make_runner(dirs[name], "bfloat16", max_tokens=128, page_size=PAGE_SIZES[name])
    records = portions("n", tokens, [70, 9, 1, 1, 2])[:5]         # a large step, then small ones
    rows = collect(records, replay(runner, records))
    layers = config["num_hidden_layers"]
    assert calls == ([4] * (layers - 1) + [3]) * 4, calls           # per small step: one chain a layer
    compare(rows, {"n": {p: plain[p] for p in rows["n"]}}, "bfloat16")
    assert not gemm._PENDING


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_that_nobody_waits_for(dtype, models):
    """Portions that want no logits are never read back, so the host prepares several steps
    while the device still works on an earlier one: held back here by a timed spin in front of
    them.  Each step's metadata must reach the device as the host wrote it for that step."""
    from rapid_llm_b200.engine.runner import StepEntry

    dirs, plains = models[dtype]
    config, weights = plains["A"]
    tokens = random_tokens(config["vocab_size"], 90, 77)
    plain = forward_logits(config, weights, tokens)
    runner = make_runner(dirs["A"], dtype, max_tokens=128, page_size=PAGE_SIZES["A"])
    cuts = [0, 7, 20, 23, 41, 52, 66, 81, 90]
    assert runner.admit("warm")               # whatever the first steps load or allocate is done before
    for begin, end in zip(cuts[:-1], cuts[1:]):
        runner.step([StepEntry("warm", tokens[begin:end], [])])
    runner.release("warm")
    assert runner.admit("r")
    torch.cuda.synchronize()
    torch.cuda._sleep(400_000_000)          # about a fifth of a second of device time
    for begin, end in zip(cuts[:-2], cuts[1:-1]):
        runner.step([StepEntry("r", tokens[begin:end], [])])
    logits = runner.step([StepEntry("r", tokens[cuts[-2]:], list(range(cuts[-1] - cuts[-2])))])
    runner.check_fault()
    got = logits.float().cpu()
    torch.testing.assert_close(got, plain[cuts[-2]:], **for_dtype(dtype))
    runner.release("r")
    runner.cache.check()


def test_window_pages_are_given_back(models):
    dirs, plains = models["float32"]
    config, _ = plains["C"]
    tokens = random_tokens(config["vocab_size"], 200, 11)
    runner = make_runner(dirs["C"], "float32", max_tokens=256, page_size=16)
    records = portions("w", tokens, [16])
    from rapid_llm_b200.replay import Replayer

    replayer = Replayer(runner)
    for record in records[:-1]:
        replayer.run_step(record)
    groups = runner.cache.groups
    windowed = [i for i, g in enumerate(groups) if g.window]
    full = [i for i, g in enumerate(groups) if not g.window]
    assert windowed and full
    pages = runner.cache.pages_of("w")
    live_window = [p for p in pages[windowed[0]] if p]
    live_full = [p for p in pages[full[0]] if p]
    assert len(live_full) == len(pages[full[0]])
    assert len(live_window) <= config["sliding_window"] // 16 + 2 < len(live_full)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(dtype, models, tmp_path):
    """``bin/trace_run`` as a user calls it: JSON lines in, ``done`` lines and .f32 files out."""
    dirs, plains = models[dtype]
    config, weights = plains["A"]
    tokens = random_tokens(config["vocab_size"], 50, 3)
    records = portions("a", tokens, [7, 2, 20])
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(dirs["A"]), "--dtype", dtype,
         "--out", str(out), "--max-tokens", "128"],
        input="".join(json.dumps(r) + "\n" for r in records), capture_output=True, text=True, timeout=600,
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for r in records for w in ("done", str(r["step"]))]
    outputs = {
        r["step"]: torch.from_numpy(np.fromfile(out / f"{r['step']}.f32", dtype="<f4").reshape(-1, config["vocab_size"]))
        for r in records
    }
    compare(collect(records, outputs), {"a": forward_logits(config, weights, tokens)}, dtype)
