"""A run order in which a layer reads another entry's cache, and runs twice.

The architecture is the test's own, put together from the stock parts: four layers, the third of which has
no key and value projections of its own (``shares_cache``); the run order is ``0, 1, 2 <- cache of entry 0,
3, 2 <- cache of entry 1``.  The framework's files do not know it.  Compared with a plain restatement (whole
sequences, no cache): whole, in a mixed trace on pages that are used again, and decoding from captured graphs,
in float32 and bfloat16, with small heads and with heads of 128 (the tensor-core attention kernels).
"""

from __future__ import annotations

import dataclasses

import pytest
import torch
from plain_qwen3 import apply_rope, causal_attention, load_model_dir, rms_norm, rope_angles, swiglu
from tolerances import for_dtype
from trace_tools import collect, mixed

pytestmark = pytest.mark.gpu

ORDER = ((0, None), (1, None), (2, 0), (3, None), (2, 1))       # (layer, the entry whose cache it reads)
SHARING_LAYER = 2


@dataclasses.dataclass(frozen=True)
class SharedCacheConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    eps: float
    theta: float
    max_positions: int
    architecture = "SharedCacheForCausalLM"
    model_type = "shared_cache_toy"

    @classmethod
    def from_dict(cls, raw, overrides=None):
        raw = dict(raw, **(overrides or {}))
        return cls(**{field.name: raw[field.name] for field in dataclasses.fields(cls)})

    def to_dict(self):
        return {"architectures": [self.architecture], "model_type": self.model_type, **dataclasses.asdict(self)}

    def to_spec(self):
        from rapid_llm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.eps})
        position = PartSpec("rope", {"head_dim": self.head_dim, "rotary_dim": self.head_dim, "theta": self.theta,
                                     "max_positions": self.max_positions})

        def attention(shares: bool) -> PartSpec:
            return PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads,
                "head_dim": self.head_dim, "position": position, "qk_norm": True, "qk_norm_eps": self.eps,
                "shares_cache": shares,
            })

        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        layers = tuple(LayerSpec("prenorm", attention(index == SHARING_LAYER), ffn, norm, f"model.layers.{index}.")
                       for index in range(4))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            layers=layers, schedule=tuple(ScheduleEntry(layer, cache_from=source) for layer, source in ORDER),
            final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": False}),
        )


CONFIGS = {
    "small_heads": SharedCacheConfig(211, 72, 120, 6, 2, 32, 1e-5, 10000.0, 256),
    "heads_of_128": SharedCacheConfig(300, 136, 264, 4, 2, 128, 1e-6, 1000000.0, 512),
}
PAGES = {"small_heads": 8, "heads_of_128": 16}


def plain_logits(config: SharedCacheConfig, weights: dict, tokens: list[int]) -> torch.Tensor:
    """The run order written out: an entry that reads another's cache attends to that entry's keys and values
    (normed and rotated as that entry made them) with queries of its own."""
    heads, kv_heads, dim = config.num_heads, config.num_kv_heads, config.head_dim
    count = len(tokens)
    positions = torch.arange(count)
    cos, sin = rope_angles(positions, dim, config.theta)
    h = weights["model.embed_tokens.weight"][tokens]
    made: list[tuple[torch.Tensor, torch.Tensor] | None] = []
    for layer, source in ORDER:
        prefix = f"model.layers.{layer}."
        x = rms_norm(h, weights[prefix + "input_layernorm.weight"], config.eps)
        q = (x @ weights[prefix + "self_attn.q_proj.weight"].T).view(count, heads, dim)
        q = apply_rope(rms_norm(q, weights[prefix + "self_attn.q_norm.weight"], config.eps), cos, sin)
        if source is None:
            k = (x @ weights[prefix + "self_attn.k_proj.weight"].T).view(count, kv_heads, dim)
            v = (x @ weights[prefix + "self_attn.v_proj.weight"].T).view(count, kv_heads, dim)
            k = apply_rope(rms_norm(k, weights[prefix + "self_attn.k_norm.weight"], config.eps), cos, sin)
            made.append((k, v))
        else:
            k, v = made[source]
            made.append(None)
        attended = causal_attention(q, k, v, dim**-0.5).reshape(count, heads * dim)
        h = h + attended @ weights[prefix + "self_attn.o_proj.weight"].T
        h = h + swiglu(rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], config.eps), weights, prefix)
    return rms_norm(h, weights["model.norm.weight"], config.eps) @ weights["lm_head.weight"].T


def compare(rows, plain, dtype, label):
    tolerance = for_dtype(dtype)
    for request_id, by_position in rows.items():
        for position, got in sorted(by_position.items()):
            try:
                torch.testing.assert_close(got, plain[request_id][position], **tolerance)
            except AssertionError as exc:
                raise AssertionError(f"{label}: request {request_id!r}, position {position}: {exc}") from None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_an_entry_reads_another_entrys_cache_and_a_layer_runs_twice(name, dtype, tmp_path):
    from rapid_llm_b200.config import EngineConfig, parse_dtype, register_architecture
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.replay import Replayer, engine_config_for
    from rapid_llm_b200.weights import write_random_model

    register_architecture(SharedCacheConfig)
    config, page = CONFIGS[name], PAGES[name]
    torch_dtype = parse_dtype(dtype)
    folder = write_random_model(tmp_path / name, config, seed=21, dtype=torch_dtype)
    _, weights = load_model_dir(folder)
    assert f"model.layers.{SHARING_LAYER}.self_attn.k_proj.weight" not in weights       # no keys of its own
    generator = torch.Generator().manual_seed(31)
    lengths = [45, 130, 22, 201, 77]
    sequences = {f"r{index}": torch.randint(0, config.vocab_size, (length,), generator=generator).tolist()
                 for index, length in enumerate(lengths)}
    plain = {rid: plain_logits(config, weights, tokens) for rid, tokens in sequences.items()}

    # mixed: portions beside decoded tokens, so few pages that they are used again
    records, peak = mixed(sequences, seed=3, max_live=3, page=page)
    runner = ModelRunner.from_folder(folder, engine_config_for(config, dtype, peak, page, 3))
    # entries 0, 1 and 3 write pages; entries 2 and 4 (the sharing layer, twice) have none of their own
    assert [cache.writes for cache in runner.layer_caches()] == [True, True, False, True, False]
    replayer, outputs = Replayer(runner), {}
    for record in records:
        out = replayer.run_step(record)
        if out is not None:
            outputs[record["step"]] = torch.from_numpy(out.copy())
        runner.cache.check()
    compare(collect(records, outputs), plain, dtype, f"{name} (mixed)")
    del runner, replayer

    # whole prompts but for their tails; the tails decoded together from captured graphs
    names, tail = ["r1", "r3"], 10
    limit = config.max_positions
    engine = EngineConfig(dtype=torch_dtype, max_seq_len=limit, page_size=page, num_pages=2 * (-(-limit // page)) + 1,
                          max_num_seqs=2, max_num_batched_tokens=limit, max_chunk_size=limit, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    for rid in names:
        assert runner.admit(rid)
        tokens = sequences[rid]
        logits = runner.step([StepEntry(rid, tokens[:-tail], list(range(len(tokens) - tail)))]).float().cpu()
        compare({rid: dict(enumerate(logits))}, plain, dtype, f"{name} (whole)")
    for offset in range(tail):
        entries = [StepEntry(rid, [sequences[rid][len(sequences[rid]) - tail + offset]], [0]) for rid in names]
        logits = runner.step_decode(entries).float().cpu()
        for row, rid in enumerate(names):
            compare({rid: {len(sequences[rid]) - tail + offset: logits[row]}}, plain, dtype, f"{name} (graph decode)")
    for rid in names:
        runner.release(rid)
    runner.check_fault()
    runner.cache.check()
