"""One layer at the widths of the large models (hidden 5120, 40 or 64 query heads over 8, head
size 128, intermediate sizes that are no power of two), bfloat16, against the plain
implementation: the tcgen05 products with their k-splits, the tcgen05 attention kernels with
groups of 5 and 8, and the library product above 64 tokens meet sizes here that the tiny
configurations never reach."""

from __future__ import annotations

import pytest
import torch
from plain_qwen3 import forward_logits, load_model_dir
from tolerances import at_scale

pytestmark = pytest.mark.gpu

WIDE = {
    "heads40_inter17408": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=17408),
    "heads64_inter25600": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600),
}


def wide_config(sizes: dict) -> dict:
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 1000, "num_hidden_layers": 1,
        "head_dim": 128, "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "tie_word_embeddings": False, "attention_bias": False, "hidden_act": "silu", "sliding_window": None,
        "use_sliding_window": False, "torch_dtype": "bfloat16", **sizes,
    }


@pytest.mark.parametrize("name", sorted(WIDE))
def test_one_wide_layer_whole_in_portions_and_decoding(name, tmp_path):
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(WIDE[name])
    folder = write_random_model(tmp_path / name, Qwen3Config.from_dict(raw), 11, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(4)
    tokens = {"a": torch.randint(0, 1000, (300,), generator=generator).tolist(),
              "b": torch.randint(0, 1000, (90,), generator=generator).tolist()}
    plain = {key: forward_logits(config, weights, ids) for key, ids in tokens.items()}

    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=512, page_size=16, num_pages=40, max_num_seqs=4,
                          max_num_batched_tokens=512, use_cuda_graph=False)
    runner = ModelRunner.from_folder(folder, engine)
    tolerance = at_scale("bfloat16", plain["a"])

    # whole: 300 tokens in one step (library products, the prompt attention kernel)
    runner.admit("a")
    places = [0, 1, 63, 64, 127, 128, 255, 256, 299]
    got = runner.step([StepEntry("a", tokens["a"], places)]).float().cpu()
    torch.testing.assert_close(got, plain["a"][places], **tolerance)
    runner.release("a")

    # portions of one beside decode tokens of the other (the streaming products, both attention kernels)
    runner.admit("a")
    runner.admit("b")
    runner.step([StepEntry("a", tokens["a"][:250], []), StepEntry("b", tokens["b"][:86], [])])
    at = {"a": 250, "b": 86}
    plan = [{"a": 47, "b": 1}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": 1, "b": 1}]
    for sizes in plan:
        entries, wanted = [], []
        for key, size in sizes.items():
            entries.append(StepEntry(key, tokens[key][at[key] : at[key] + size], [size - 1]))
            at[key] += size
            wanted.append(plain[key][at[key] - 1])
        got = runner.step(entries).float().cpu()
        torch.testing.assert_close(got, torch.stack(wanted), **tolerance)
    runner.check_fault()
    assert at == {"a": 300, "b": 90}


def test_a_step_of_more_than_a_thousand_tokens_at_the_widths_of_a_large_model(tmp_path):
    """Two prompts of 700 and 400 tokens in one step at hidden 5120 and an intermediate size of 17,408: from 1,024
    tokens on the gate/up product applies its activation itself, on pairs of CTAs, here over 136 weight tiles and
    five token tiles of which the last is ragged and holds the end of one request and nothing after it."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.ops import gemm
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(WIDE["heads40_inter17408"])
    raw["max_position_embeddings"] = 1024
    folder = write_random_model(tmp_path / "wide", Qwen3Config.from_dict(raw), 12, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(9)
    tokens = {"a": torch.randint(0, 1000, (700,), generator=generator).tolist(),
              "b": torch.randint(0, 1000, (400,), generator=generator).tolist()}
    assert sum(len(ids) for ids in tokens.values()) >= gemm.PAIR_GATED_MIN_TOKENS
    plain = {key: forward_logits(config, weights, ids) for key, ids in tokens.items()}
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=1024, page_size=16, num_pages=80, max_num_seqs=2,
                          max_num_batched_tokens=1536, max_chunk_size=1536, use_cuda_graph=False)
    runner = ModelRunner.from_folder(folder, engine)
    runner.admit("a")
    runner.admit("b")
    places = {"a": [0, 255, 256, 511, 699], "b": [0, 67, 68, 399]}       # 68: the first row of the last token tile
    got = runner.step([StepEntry("a", tokens["a"], places["a"]), StepEntry("b", tokens["b"], places["b"])]).float().cpu()
    want = torch.cat([plain["a"][places["a"]], plain["b"][places["b"]]])
    torch.testing.assert_close(got, want, **at_scale("bfloat16", plain["a"]))
    runner.check_fault()


def test_a_long_context_with_heads_of_128(tmp_path):
    """3,300 tokens through two narrow layers with heads of 128: prompt portions whose tiles look
    back over thousands of cached keys, then single tokens whose key range is split over a
    cluster, against the plain implementation."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(dict(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, intermediate_size=512))
    raw.update(num_hidden_layers=2, vocab_size=500, max_position_embeddings=4096)
    folder = write_random_model(tmp_path / "long", Qwen3Config.from_dict(raw), 13, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    tokens = torch.randint(0, 500, (3300,), generator=torch.Generator().manual_seed(6)).tolist()
    plain = forward_logits(config, weights, tokens)
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=4096, page_size=16, num_pages=260, max_num_seqs=2,
                          max_num_batched_tokens=1024, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    tolerance = at_scale("bfloat16", plain)
    runner.admit("r")
    at = 0
    for size in (1024, 1024, 1000, 246):
        places = [0, size // 2, size - 1]
        got = runner.step([StepEntry("r", tokens[at : at + size], places)]).float().cpu()
        torch.testing.assert_close(got, plain[[at + p for p in places]], **tolerance)
        at += size
    for _ in range(6):
        got = runner.step_decode([StepEntry("r", tokens[at : at + 1], [0])]).float().cpu()
        torch.testing.assert_close(got, plain[at : at + 1], **tolerance)
        at += 1
    runner.check_fault()
    assert at == 3300


def test_single_tokens_far_into_their_context_beside_a_prompt_portion(tmp_path):
    """A step of prompt portions (which the tcgen05 kernel takes unsplit) beside single tokens of requests that are
    thousands of tokens into their contexts: the single tokens' tiles get key ranges of their own, merged inside the
    decode kernel's clusters (ten ranges for one such request, six for two), and both kinds of rows agree with the
    plain implementation."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.parts.base import StepShape
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(dict(hidden_size=256, num_attention_heads=16, num_key_value_heads=8, intermediate_size=512))
    raw.update(num_hidden_layers=2, vocab_size=500, max_position_embeddings=4096)
    folder = write_random_model(tmp_path / "mixed", Qwen3Config.from_dict(raw), 14, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(16)
    tokens = {"far": torch.randint(0, 500, (3010,), generator=generator).tolist(),
              "deep": torch.randint(0, 500, (1500,), generator=generator).tolist(),
              "new": torch.randint(0, 500, (1800,), generator=generator).tolist()}
    plain = {name: forward_logits(config, weights, ids) for name, ids in tokens.items()}
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=4096, page_size=16, num_pages=400, max_num_seqs=3,
                          max_num_batched_tokens=1024, use_cuda_graph=False)
    runner = ModelRunner.from_folder(folder, engine)
    tolerance = at_scale("bfloat16", plain["far"])
    at = {"far": 3000, "deep": 1494, "new": 0}
    for name in ("far", "deep"):
        runner.admit(name)
        fed = 0
        while fed < at[name]:
            size = min(1000, at[name] - fed)
            runner.step([StepEntry(name, tokens[name][fed : fed + size], [])])
            fed += size
    runner.admit("new")
    (planner,) = runner.model.step_planners()      # what the step function asks for the same step
    plans = []
    for portion, decoding in ((600, ("far",)), (600, ("far", "deep")), (600, ("far", "deep"))):
        entries = [StepEntry("new", tokens["new"][at["new"] : at["new"] + portion], [portion - 1])]
        wanted, starts = [plain["new"][at["new"] + portion - 1]], [at["new"]]
        at["new"] += portion
        for name in decoding:
            entries.append(StepEntry(name, tokens[name][at[name] : at[name] + 1], [0]))
            wanted.append(plain[name][at[name]])
            starts.append(at[name])
            at[name] += 1
        got = runner.step(entries).float().cpu()
        torch.testing.assert_close(got, torch.stack(wanted), **tolerance)
        plan = planner.plan(StepShape([len(entry.tokens) for entry in entries], starts, False, page_size=16))
        plans.append((plan["splits"], plan["decode_splits"]))
    assert plans == [(1, 10), (1, 6), (1, 6)]
    runner.check_fault()


def test_a_window_on_one_layer_with_heads_of_128(tmp_path):
    """Two layers with heads of 128, the second with a window of 200 keys: the tcgen05 kernels mask
    the window's edge, the windowed group gives pages back as the window passes them."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=384))
    raw.update(num_hidden_layers=2, vocab_size=400, max_position_embeddings=1024,
               use_sliding_window=True, sliding_window=200, max_window_layers=1)
    folder = write_random_model(tmp_path / "window", Qwen3Config.from_dict(raw), 14, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    tokens = torch.randint(0, 400, (900,), generator=torch.Generator().manual_seed(7)).tolist()
    plain = forward_logits(config, weights, tokens)
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=1024, page_size=16, num_pages=70, max_num_seqs=2,
                          max_num_batched_tokens=512, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    assert len(runner.cache.groups) == 2
    tolerance = at_scale("bfloat16", plain)
    runner.admit("r")
    at = 0
    for size in (300, 7, 512, 61):
        places = [0, size - 1]
        got = runner.step([StepEntry("r", tokens[at : at + size], places)]).float().cpu()
        torch.testing.assert_close(got, plain[[at + p for p in places]], **tolerance)
        at += size
    for _ in range(20):
        got = runner.step_decode([StepEntry("r", tokens[at : at + 1], [0])]).float().cpu()
        torch.testing.assert_close(got, plain[at : at + 1], **tolerance)
        at += 1
    runner.check_fault()
    runner.cache.check()
    held = sorted(sum(1 for p in pages if p) for pages in runner.cache.pages_of("r"))
    assert held[1] >= 56 and held[0] <= 15               # all keys in one group, a window of them in the other


def test_graph_decode_of_three_requests_padded_to_a_bucket_of_four(tmp_path):
    """Heads of 128, three requests decoded together from a captured graph whose batch is padded
    with a row on the null page; then two of them, after the third has ended."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=1, intermediate_size=384))
    raw.update(num_hidden_layers=2, vocab_size=400, max_position_embeddings=512)
    folder = write_random_model(tmp_path / "bucket", Qwen3Config.from_dict(raw), 15, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(8)
    tokens = {name: torch.randint(0, 400, (count,), generator=generator).tolist()
              for name, count in (("a", 48), ("b", 181), ("c", 310))}
    plain = {name: forward_logits(config, weights, ids) for name, ids in tokens.items()}
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=512, page_size=16, num_pages=48, max_num_seqs=4,
                          max_num_batched_tokens=512, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    tolerance = at_scale("bfloat16", plain["c"])
    at = {}
    for name, ids in tokens.items():
        runner.admit(name)
        at[name] = len(ids) - 8
        runner.step([StepEntry(name, ids[: at[name]], [])])
    live = ["a", "b", "c"]
    for step in range(8):
        if step == 5:
            runner.release("b")
            live.remove("b")
        entries = [StepEntry(name, tokens[name][at[name] : at[name] + 1], [0]) for name in live]
        got = runner.step_decode(entries).float().cpu()
        want = torch.stack([plain[name][at[name]] for name in live])
        torch.testing.assert_close(got, want, **tolerance)
        for name in live:
            at[name] += 1
    runner.check_fault()
    runner.cache.check()


def test_graph_decode_across_the_context_lengths_at_which_its_launches_change(tmp_path):
    """Heads of 128: a decode tile is cut into no more key ranges than the context has blocks of 128 keys
    (1, 2, 4, 8, then what the GPU's clusters allow), so a request that grows from 100 to 1,100 tokens
    passes through several captured graphs of one bucket; the steps before, at and after every change are
    compared with the plain implementation, and a replayed graph with a freshly captured one."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=384))
    raw.update(num_hidden_layers=2, vocab_size=400, max_position_embeddings=1280)
    folder = write_random_model(tmp_path / "classes", Qwen3Config.from_dict(raw), 16, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(9)
    ids = torch.randint(0, 400, (1100,), generator=generator).tolist()
    plain = forward_logits(config, weights, ids)
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=1280, page_size=16, num_pages=96, max_num_seqs=2,
                          max_num_batched_tokens=1280, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    tolerance = at_scale("bfloat16", plain)
    runner.admit("a")
    runner.step([StepEntry("a", ids[:100], [])])
    seen = []
    for at in range(100, 1100):
        got = runner.step_decode([StepEntry("a", ids[at : at + 1], [0])]).float().cpu()
        torch.testing.assert_close(got[0], plain[at], **tolerance)
        splits = sorted({value for _, constants in runner._graphs for _, name, value in constants if name == "splits"})
        if not seen or seen[-1] != splits:
            seen.append(splits)
    runner.check_fault()
    runner.cache.check()
    assert seen[-1][:4] == [1, 2, 4, 8] and len(seen) >= 4          # one graph per class, each used again after its capture
    assert {bucket for bucket, _ in runner._graphs} == {1}


def test_graph_decode_with_a_cluster_of_sixteen_key_ranges(tmp_path):
    """Past 2,048 tokens a single request's decode tile is cut into as many key ranges as the GPU runs clusters of
    (16 CTAs with two kv heads: a cluster size that has to be asked for), captured and replayed."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=384))
    raw.update(num_hidden_layers=2, vocab_size=400, max_position_embeddings=2304)
    folder = write_random_model(tmp_path / "sixteen", Qwen3Config.from_dict(raw), 17, dtype=torch.bfloat16)
    config, weights = load_model_dir(folder)
    ids = torch.randint(0, 400, (2200,), generator=torch.Generator().manual_seed(10)).tolist()
    tail = 6
    plain = forward_logits(config, weights, ids, rows=range(len(ids) - tail, len(ids)))
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=2304, page_size=16, num_pages=160, max_num_seqs=2,
                          max_num_batched_tokens=2304, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    runner.admit("a")
    runner.step([StepEntry("a", ids[:-tail], [])])
    got = []
    for at in range(len(ids) - tail, len(ids)):
        got.append(runner.step_decode([StepEntry("a", ids[at : at + 1], [0])]).float().cpu()[0])
    runner.check_fault()
    torch.testing.assert_close(torch.stack(got), plain, **at_scale("bfloat16", plain))
    splits = {value for _, constants in runner._graphs for _, name, value in constants if name == "splits"}
    assert splits and max(splits) > 8, splits


def test_the_same_steps_give_the_same_bits(tmp_path):
    """Reduction orders are fixed (cluster sums in rank order, split key ranges merged in order, no
    atomics on values): two engines fed the same steps return identical logits, bit for bit."""
    from rapid_llm_b200.config import EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    raw = wide_config(dict(hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, intermediate_size=2816))
    raw.update(num_hidden_layers=2, vocab_size=3001, max_position_embeddings=1024)
    folder = write_random_model(tmp_path / "bits", Qwen3Config.from_dict(raw), 16, dtype=torch.bfloat16)
    generator = torch.Generator().manual_seed(9)
    tokens = {name: torch.randint(0, 3001, (count,), generator=generator).tolist() for name, count in (("a", 700), ("b", 90))}

    def run():
        engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=1024, page_size=16, num_pages=64, max_num_seqs=4,
                              max_num_batched_tokens=512, use_cuda_graph=True)
        runner = ModelRunner.from_folder(folder, engine)
        outputs = []
        runner.admit("a"), runner.admit("b")
        outputs.append(runner.step([StepEntry("a", tokens["a"][:400], [399]), StepEntry("b", tokens["b"][:60], [0, 59])]).clone())
        outputs.append(runner.step([StepEntry("a", tokens["a"][400:690], [0, 289]), StepEntry("b", tokens["b"][60:61], [0])]).clone())
        at = {"a": 690, "b": 61}
        for _ in range(6):
            entries = [StepEntry(name, tokens[name][at[name] : at[name] + 1], [0]) for name in ("a", "b")]
            outputs.append(runner.step_decode(entries).clone())
            for name in at:
                at[name] += 1
        runner.check_fault()
        return outputs

    first, second = run(), run()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
