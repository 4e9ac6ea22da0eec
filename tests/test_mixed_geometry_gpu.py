"""Layers whose attention differs in every size: the cache manager keeps a group of pages for each geometry.

The architecture is the test's own, put together from the stock parts: three layers with (heads, kv heads, head
size) of (6, 2, 32), (4, 1, 64) and (8, 4, 16), the last with a window, and feed-forwards of three intermediate
sizes.  Nothing in the framework's files knows it.  Whole sequences, a mixed trace on few pages and decoding from
captured graphs against a plain restatement, in float32 and bfloat16.
"""

from __future__ import annotations

import dataclasses

import pytest
import torch
from plain_qwen3 import apply_rope, causal_attention, load_model_dir, rms_norm, rope_angles, swiglu
from tolerances import for_dtype
from trace_tools import collect, mixed

pytestmark = pytest.mark.gpu

GEOMETRY = ((6, 2, 32, 0, 96), (4, 1, 64, 0, 160), (8, 4, 16, 37, 72))    # heads, kv heads, head size, window, intermediate
HIDDEN, VOCAB, EPS, THETA, POSITIONS = 88, 263, 1e-5, 10000.0, 256


@dataclasses.dataclass(frozen=True)
class MixedGeometryConfig:
    vocab_size: int = VOCAB
    hidden_size: int = HIDDEN
    architecture = "MixedGeometryForCausalLM"
    model_type = "mixed_geometry_toy"

    @classmethod
    def from_dict(cls, raw, overrides=None):
        raw = dict(raw, **(overrides or {}))
        return cls(raw["vocab_size"], raw["hidden_size"])

    def to_dict(self):
        return {"architectures": [self.architecture], "model_type": self.model_type, **dataclasses.asdict(self)}

    def to_spec(self):
        from rapid_llm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": EPS})
        layers = []
        for index, (heads, kv_heads, dim, window, inter) in enumerate(GEOMETRY):
            position = PartSpec("rope", {"head_dim": dim, "rotary_dim": dim, "theta": THETA, "max_positions": POSITIONS})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": dim,
                "position": position, "qk_norm": True, "qk_norm_eps": EPS, "window": window,
            })
            ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": inter})
            layers.append(LayerSpec("prenorm", mixer, ffn, norm, f"model.layers.{index}."))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size, max_positions=POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": True}),
        )


def plain_logits(weights: dict, tokens: list[int]) -> torch.Tensor:
    count = len(tokens)
    positions = torch.arange(count)
    h = weights["model.embed_tokens.weight"][tokens]
    for index, (heads, kv_heads, dim, window, _) in enumerate(GEOMETRY):
        prefix = f"model.layers.{index}."
        cos, sin = rope_angles(positions, dim, THETA)
        x = rms_norm(h, weights[prefix + "input_layernorm.weight"], EPS)
        q = (x @ weights[prefix + "self_attn.q_proj.weight"].T).view(count, heads, dim)
        k = (x @ weights[prefix + "self_attn.k_proj.weight"].T).view(count, kv_heads, dim)
        v = (x @ weights[prefix + "self_attn.v_proj.weight"].T).view(count, kv_heads, dim)
        q = apply_rope(rms_norm(q, weights[prefix + "self_attn.q_norm.weight"], EPS), cos, sin)
        k = apply_rope(rms_norm(k, weights[prefix + "self_attn.k_norm.weight"], EPS), cos, sin)
        attended = causal_attention(q, k, v, dim**-0.5, window).reshape(count, heads * dim)
        h = h + attended @ weights[prefix + "self_attn.o_proj.weight"].T
        h = h + swiglu(rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], EPS), weights, prefix)
    return rms_norm(h, weights["model.norm.weight"], EPS) @ weights["model.embed_tokens.weight"].T


def compare(rows, plain, dtype, label):
    tolerance = for_dtype(dtype)
    for request_id, by_position in rows.items():
        for position, got in sorted(by_position.items()):
            try:
                torch.testing.assert_close(got, plain[request_id][position], **tolerance)
            except AssertionError as exc:
                raise AssertionError(f"{label}: request {request_id!r}, position {position}: {exc}") from None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_layer_has_a_geometry_and_a_group_of_pages_of_its_own(dtype, tmp_path):
    from rapid_llm_b200.config import EngineConfig, parse_dtype, register_architecture
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.replay import Replayer, engine_config_for
    from rapid_llm_b200.weights import write_random_model

    register_architecture(MixedGeometryConfig)
    config, page = MixedGeometryConfig(), 8
    torch_dtype = parse_dtype(dtype)
    folder = write_random_model(tmp_path / "model", config, seed=41, dtype=torch_dtype)
    _, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(43)
    lengths = [52, 140, 19, 230, 88]
    sequences = {f"r{index}": torch.randint(0, VOCAB, (length,), generator=generator).tolist()
                 for index, length in enumerate(lengths)}
    plain = {rid: plain_logits(weights, tokens) for rid, tokens in sequences.items()}

    records, peak = mixed(sequences, seed=5, max_live=3, page=page)
    runner = ModelRunner.from_folder(folder, engine_config_for(config, dtype, peak, page, 3))
    groups = runner.cache.groups
    assert len(groups) == 3 and sorted(group.entries for group in groups) == [(0,), (1,), (2,)]
    assert sorted(int(group.window) for group in groups) == [0, 0, 37]
    replayer, outputs = Replayer(runner), {}
    for record in records:
        out = replayer.run_step(record)
        if out is not None:
            outputs[record["step"]] = torch.from_numpy(out.copy())
        runner.cache.check()
    compare(collect(records, outputs), plain, dtype, "mixed")
    del runner, replayer

    names, tail = ["r1", "r3"], 9
    engine = EngineConfig(dtype=torch_dtype, max_seq_len=POSITIONS, page_size=page, num_pages=2 * (POSITIONS // page) + 1,
                          max_num_seqs=2, max_num_batched_tokens=POSITIONS, max_chunk_size=POSITIONS, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    for rid in names:
        assert runner.admit(rid)
        tokens = sequences[rid]
        logits = runner.step([StepEntry(rid, tokens[:-tail], list(range(len(tokens) - tail)))]).float().cpu()
        compare({rid: dict(enumerate(logits))}, plain, dtype, "whole")
    for offset in range(tail):
        entries = [StepEntry(rid, [sequences[rid][len(sequences[rid]) - tail + offset]], [0]) for rid in names]
        logits = runner.step_decode(entries).float().cpu()
        for row, rid in enumerate(names):
            compare({rid: {len(sequences[rid]) - tail + offset: logits[row]}}, plain, dtype, "graph decode")
    for rid in names:
        runner.release(rid)
    runner.check_fault()
    runner.cache.check()
