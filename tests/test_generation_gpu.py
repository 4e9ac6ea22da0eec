"""Generation through the Python entry point against the plain implementation."""

from __future__ import annotations

import pytest
import torch
from plain_qwen3 import forward_logits, greedy_generate, sample_token
from tiny_configs import PAGE_SIZES

pytestmark = pytest.mark.gpu


def random_prompts(vocab, lengths, seed):
    generator = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in lengths]


def make_llm(folder, dtype, name, **overrides):
    from rapid_llm_b200 import LLM

    values = dict(dtype=dtype, max_seq_len=128, max_gpu_num_blocks=64, page_size=PAGE_SIZES[name],
                  max_num_seqs=4, max_chunk_size=13, max_num_batched_tokens=64)
    values.update(overrides)
    return LLM(folder, **values)


def test_greedy_float32_equals_plain(tiny_dirs, tiny_plain):
    from rapid_llm_b200 import SamplingParams

    config, weights = tiny_plain["A"]
    prompts = random_prompts(config["vocab_size"], [5, 17, 33], 1)
    llm = make_llm(tiny_dirs["A"], "float32", "A")
    outputs = llm.generate(prompts, SamplingParams.greedy(max_gen_len=8))
    for prompt, output in zip(prompts, outputs):
        assert output.token_ids == greedy_generate(config, weights, prompt, 8)
        assert output.outputs[0].finish_reason == "length" and output.prompt_token_ids == prompt
    llm.runner.cache.check()
    assert llm.runner.cache.num_free_slots == 4


@pytest.mark.parametrize("use_graph", [False, True])
def test_greedy_bfloat16_picks_a_maximum_of_the_plain_logits(tiny_dirs_bf16, tiny_plain_bf16, use_graph):
    from rapid_llm_b200 import SamplingParams

    config, weights = tiny_plain_bf16["B"]
    prompts = random_prompts(config["vocab_size"], [1, 7, 31, 64, 100], 2)
    llm = make_llm(tiny_dirs_bf16["B"], "bfloat16", "B", max_seq_len=160, use_cuda_graph=use_graph)
    outputs = llm.generate(prompts, SamplingParams.greedy(max_gen_len=12))
    for prompt, output in zip(prompts, outputs):
        tokens = output.token_ids
        assert len(tokens) == 12
        logits = forward_logits(config, weights, prompt + tokens)
        for index, token in enumerate(tokens):
            row = logits[len(prompt) - 1 + index]
            assert float(row.max() - row[token]) < 2e-2


def test_graph_and_eager_decode_agree(tiny_dirs):
    from rapid_llm_b200 import SamplingParams

    prompts = random_prompts(384, [9, 30, 3], 5)
    eager = make_llm(tiny_dirs["B"], "float32", "B", use_cuda_graph=False).generate(prompts, SamplingParams.greedy(max_gen_len=20))
    graph = make_llm(tiny_dirs["B"], "float32", "B", use_cuda_graph=True).generate(prompts, SamplingParams.greedy(max_gen_len=20))
    assert [o.token_ids for o in eager] == [o.token_ids for o in graph]


def test_the_command_line_from_a_folder_to_token_ids(tiny_dirs, tiny_plain, tmp_path):
    """``python -m rapid_llm_b200.cli batch --prompt-ids-file``: a model folder and a file of prompts in, the
    plain implementation's greedy tokens out; with ``--stop-token-ids`` a request ends at that token."""
    import subprocess
    import sys
    from pathlib import Path

    config, weights = tiny_plain["A"]
    prompts = random_prompts(config["vocab_size"], [5, 17, 33], 1)
    ids_file = tmp_path / "prompts.txt"
    ids_file.write_text("".join(" ".join(map(str, prompt)) + "\n" for prompt in prompts))
    root = Path(__file__).resolve().parents[1]
    base = [sys.executable, "-m", "rapid_llm_b200.cli", "batch", "--model-dir", str(tiny_dirs["A"]), "--dtype", "float32",
            "--prompt-ids-file", str(ids_file), "--temperature", "0", "--repetition-penalty", "1.0", "--max-gen-len", "8",
            "--max-seq-len", "128", "--max-gpu-num-blocks", "32", "--max-num-seqs", "4", "--max-chunk-size", "13",
            "--max-num-batched-tokens", "64"]

    def run(*extra):
        done = subprocess.run(base + list(extra), cwd=root, capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        blocks = done.stdout.split("--- [")[1:]           # "0] reason ---\n<ids or nothing>\n"
        reasons = [block.split()[1] for block in blocks]
        tokens = [[int(t) for t in block.split("---", 1)[1].split()] for block in blocks]
        return reasons, tokens

    want = [greedy_generate(config, weights, prompt, 8) for prompt in prompts]
    reasons, tokens = run()
    assert tokens == want and reasons == ["length"] * 3
    stop = want[1][-1]                # wherever it first shows in a request's tokens, the request ends before it
    reasons, tokens = run("--stop-token-ids", f"{stop}, 100000")
    for reason, got, full in zip(reasons, tokens, want):
        cut = full.index(stop) if stop in full else len(full)
        assert got == full[:cut] and reason == ("eos" if stop in full else "length")


def test_the_pool_is_sized_from_free_memory_when_no_size_is_given(tiny_dirs, tiny_plain):
    """Without ``max_gpu_num_blocks`` the pool takes what the slots can hold at full length (a tiny model on an
    empty GPU is far from the memory limit), and generation runs on it."""
    from rapid_llm_b200 import SamplingParams

    config, weights = tiny_plain["A"]
    llm = make_llm(tiny_dirs["A"], "float32", "A", max_gpu_num_blocks=None, max_num_seqs=3)
    pool = llm.runner.cache.pools[0]
    assert pool.num_pages == 3 * (128 // PAGE_SIZES["A"])
    prompt = random_prompts(config["vocab_size"], [11], 4)[0]
    assert llm.generate([prompt], SamplingParams.greedy(max_gen_len=5))[0].token_ids == greedy_generate(config, weights, prompt, 5)


def test_a_token_budget_below_the_number_of_slots(tiny_dirs, tiny_plain):
    """Six tokens a step and eight slots: five requests decoding from a graph pad to six rows, within the
    budget (the next power of two would not fit)."""
    from rapid_llm_b200 import SamplingParams

    config, weights = tiny_plain["A"]
    prompts = random_prompts(config["vocab_size"], [2, 3, 2, 2, 3], 8)
    llm = make_llm(tiny_dirs["A"], "float32", "A", max_num_seqs=8, max_num_batched_tokens=6, max_chunk_size=6,
                   use_cuda_graph=True)
    outputs = llm.generate(prompts, SamplingParams.greedy(max_gen_len=24))
    for prompt, output in zip(prompts, outputs):
        assert output.token_ids == greedy_generate(config, weights, prompt, 24)
    buckets = {bucket for bucket, _ in llm.runner._graphs}
    assert 6 in buckets and 8 not in buckets


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(tiny_dirs, tiny_plain):
    from rapid_llm_b200 import SamplingParams

    config, weights = tiny_plain["B"]
    prompts = random_prompts(config["vocab_size"], [1, 7, 31, 64, 100], 3)
    params = [SamplingParams(temperature=0.7, top_p=0.9, repetition_penalty=1.1, max_gen_len=12, seed=50 + i) for i in range(5)]
    llm = make_llm(tiny_dirs["B"], "float32", "B", max_seq_len=160)
    together = llm.generate(prompts, params)
    alone = [llm.generate([p], [sp])[0] for p, sp in zip(prompts, params)]
    assert [o.token_ids for o in together] == [o.token_ids for o in alone]
    # teacher-forced check of every draw against the plain sampler
    agree = total = 0
    for prompt, output, sp in zip(prompts, together, params):
        tokens = output.token_ids
        logits = forward_logits(config, weights, prompt + tokens)
        for index, token in enumerate(tokens):
            want = sample_token(logits[len(prompt) - 1 + index], 0.7, 0.9, 1.1, tokens[:index], sp.seed, index)
            agree += int(want == token)
            total += 1
    assert agree >= total - 2, (agree, total)


def test_eviction_under_a_small_pool_does_not_change_tokens(tiny_dirs):
    from rapid_llm_b200 import SamplingParams

    prompts = random_prompts(256, [30, 20, 25], 4)
    roomy = make_llm(tiny_dirs["A"], "float32", "A").generate(prompts, SamplingParams.greedy(max_gen_len=30))
    tight_llm = make_llm(tiny_dirs["A"], "float32", "A", max_gpu_num_blocks=8)
    tight = tight_llm.generate(prompts, SamplingParams.greedy(max_gen_len=30))
    assert [o.token_ids for o in roomy] == [o.token_ids for o in tight]
    assert tight_llm.scheduler.num_preemptions >= 1
    tight_llm.runner.cache.check()


def test_stop_token_ends_a_request(tiny_dirs, tiny_plain):
    from rapid_llm_b200 import LLM, SamplingParams

    config, weights = tiny_plain["A"]
    prompt = random_prompts(256, [12], 6)[0]
    free = greedy_generate(config, weights, prompt, 6)
    llm = LLM(tiny_dirs["A"], dtype="float32", max_seq_len=128, max_gpu_num_blocks=16, stop_token_ids=[free[3]])
    output = llm.generate([prompt], SamplingParams.greedy(max_gen_len=6))[0]
    first_stop = free.index(free[3])
    assert output.token_ids == free[:first_stop] and output.outputs[0].finish_reason == "eos"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_does_not_change_a_token(tiny_dirs, tiny_dirs_bf16, dtype):
    """Greedy and seeded temperature requests, a stop token, a pool small enough to evict: the same
    tokens whether the scheduler reads every step's ids before planning the next or runs ahead."""
    from rapid_llm_b200 import SamplingParams

    folder = (tiny_dirs if dtype == "float32" else tiny_dirs_bf16)["B"]
    prompts = random_prompts(384, [1, 7, 31, 64, 40, 3], 5)
    params = [SamplingParams.greedy(max_gen_len=20), SamplingParams(temperature=0.7, top_p=0.9, repetition_penalty=1.0, max_gen_len=15, seed=3),
              SamplingParams.greedy(max_gen_len=12), SamplingParams(temperature=1.0, top_p=1.0, repetition_penalty=1.0, max_gen_len=9, seed=8),
              SamplingParams.greedy(max_gen_len=30), SamplingParams.greedy(max_gen_len=25)]
    results = {}
    for ahead in (False, True):
        llm = make_llm(folder, dtype, "B", max_gpu_num_blocks=30, run_ahead=ahead)
        # whatever the second request samples first becomes a stop token for everybody
        probe = llm.generate([prompts[1]], [params[1]])[0].token_ids
        llm.scheduler.stop_token_ids = {probe[4]}
        outputs = llm.generate(prompts, params)
        results[ahead] = [(o.token_ids, o.outputs[0].finish_reason) for o in outputs]
        llm.runner.cache.check()
        assert llm.runner.cache.num_free_slots == 4 and llm.scheduler._inflight is None
    assert results[True] == results[False]
    assert any(reason == "eos" for _, reason in results[True])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_many_requests_under_pressure_equal_plain(tiny_dirs, tiny_plain, name):
    """Twenty requests of every length through four slots and a pool that holds two of the longest:
    portions beside decoded tokens, evictions, pages and slots used again, graphs and run-ahead on.
    Every request's greedy tokens are the plain implementation's."""
    from rapid_llm_b200 import SamplingParams

    config, weights = tiny_plain[name]
    generator = torch.Generator().manual_seed(99)
    lengths = torch.randint(1, 90, (20,), generator=generator).tolist()
    budgets = torch.randint(1, 24, (20,), generator=generator).tolist()
    prompts = random_prompts(config["vocab_size"], lengths, 17)
    page = PAGE_SIZES[name]
    llm = make_llm(tiny_dirs[name], "float32", name, max_gpu_num_blocks=2 * (-(-128 // page)) + 1,
                   max_chunk_size=29, max_num_batched_tokens=48, use_cuda_graph=True, run_ahead=True)
    outputs = llm.generate(prompts, [SamplingParams.greedy(max_gen_len=n) for n in budgets])
    for prompt, budget, output in zip(prompts, budgets, outputs):
        assert output.token_ids == greedy_generate(config, weights, prompt, budget), (len(prompt), budget)
    llm.runner.cache.check()
    assert llm.runner.cache.num_free_slots == 4
    assert llm.scheduler.num_preemptions >= 1


def test_streaming_yields_the_tokens_of_generate_piece_by_piece(tiny_dirs):
    from rapid_llm_b200 import SamplingParams

    prompts = random_prompts(256, [9, 40, 3], 8)
    params = [SamplingParams.greedy(max_gen_len=n) for n in (12, 5, 20)]
    llm = make_llm(tiny_dirs["A"], "float32", "A")
    whole = [o.token_ids for o in llm.generate(prompts, params)]
    pieces = [[] for _ in prompts]
    yields = 0
    for gained in llm.stream(prompts, params):
        assert len(gained) == len(prompts) and any(gained)
        for mine, new in zip(pieces, gained):
            mine.extend(new)
        yields += 1
    assert pieces == whole and yields >= 12
    assert all(token >= 0 for mine in pieces for token in mine)
    llm.runner.cache.check()
    assert llm.runner.cache.num_free_slots == 4


def test_a_scheduler_from_a_model_folder_steps_requests_by_hand(tiny_dirs, tiny_plain):
    """The reference's other way in: ``Scheduler.from_pretrained``, ``add_request``, ``step``."""
    from rapid_llm_b200.engine import Scheduler

    config, weights = tiny_plain["A"]
    prompt = random_prompts(256, [21], 12)[0]
    scheduler = Scheduler.from_pretrained(tiny_dirs["A"], dtype="float32", max_seq_len=128, max_gpu_num_blocks=16,
                                          page_size=PAGE_SIZES["A"], max_num_seqs=2, max_chunk_size=8)
    from rapid_llm_b200 import SamplingParams
    request = scheduler.add_request("", SamplingParams.greedy(max_gen_len=6), prompt_token_ids=prompt)
    steps = 0
    while scheduler.has_unfinished_requests():
        scheduler.step()
        steps += 1
    assert request.output_token_ids == greedy_generate(config, weights, prompt, 6) and steps >= 3 + 6
