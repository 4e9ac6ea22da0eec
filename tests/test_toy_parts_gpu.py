"""Toy parts defined here, outside the framework: a feed-forward that routes every token to one
of several experts and a position encoding of its own (interpolated positions, a partial
rotation).  Both are registered, named by a configuration layer by layer beside the stock
parts, given random weights, loaded and stepped without a change to the framework's files, and
compared with a plain restatement built from the plain implementation's functions."""

from __future__ import annotations

import dataclasses

import pytest
import torch
from plain_qwen3 import apply_rope, causal_attention, rms_norm, rope_angles, swiglu
from tolerances import for_dtype

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, VOCAB, EXPERTS, INNER = 48, 6, 2, 32, 131, 3, 40
ROTARY, SCALE, THETA, EPS, POSITIONS = 16, 4.0, 5000.0, 1e-5, 96


def register_toys():
    from rapid_llm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from rapid_llm_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding, TensorSpec

    @FEED_FORWARDS.register("toy_routed")
    class ToyRouted(FeedForward):
        """y = p_e * down_e(relu(up_e x)) with e the expert of the largest router logit and p its
        softmax probability."""

        def __init__(self, *, hidden_size, inner_size, experts, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.experts = experts
            self.router = self.new_storage((experts, hidden_size), "matrix")
            self.up = [self.new_storage((inner_size, hidden_size), "matrix") for _ in range(experts)]
            self.down = [self.new_storage((hidden_size, inner_size), "matrix") for _ in range(experts)]
            self.shapes = {"router.weight": (experts, hidden_size)}
            for e in range(experts):
                self.shapes[f"experts.{e}.up.weight"] = (inner_size, hidden_size)
                self.shapes[f"experts.{e}.down.weight"] = (hidden_size, inner_size)

        def tensor_specs(self):
            return {name: TensorSpec(shape) for name, shape in self.shapes.items()}

        def load_tensor(self, name, tensor):
            if name == "router.weight":
                self.router.copy_(tensor)
            else:
                _, index, which, _ = name.split(".")
                (self.up if which == "up" else self.down)[int(index)].copy_(tensor)

        def forward(self, x, batch):
            logits = x.float() @ self.router.float().T
            probability, expert = torch.softmax(logits, dim=-1).max(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.experts):
                rows = torch.nonzero(expert == e).flatten()
                if rows.numel():
                    hidden = torch.relu(x[rows].float() @ self.up[e].float().T)
                    out[rows] = (probability[rows, None] * (hidden @ self.down[e].float().T)).to(x.dtype)
            return out

    @POSITION_ENCODINGS.register("toy_interpolated")
    class ToyInterpolated(PositionEncoding):
        """Rotation by the angles of position / scale over the first ``rotary_dim`` sizes of a head."""

        def __init__(self, *, rotary_dim, theta, scale, max_positions, dtype, device, head_dim=None):
            super().__init__(dtype=dtype, device=device)
            cos, sin = rope_angles(torch.arange(max_positions) / scale, rotary_dim, theta)
            self.cos, self.sin = cos.to(self.device).contiguous(), sin.to(self.device).contiguous()

        def tables(self):
            return self.cos, self.sin

    @dataclasses.dataclass(frozen=True)
    class ToyPartsConfig:
        vocab_size: int = VOCAB
        architecture = "ToyPartsForCausalLM"
        model_type = "toy_parts"

        @classmethod
        def from_dict(cls, raw, overrides=None):
            return cls(dict(raw, **(overrides or {}))["vocab_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": self.model_type, "vocab_size": self.vocab_size}

        def to_spec(self):
            norm = PartSpec("rmsnorm", {"size": HIDDEN, "eps": EPS})

            def attention(position):
                return PartSpec("gqa_attention", {
                    "hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
                    "position": position, "qk_norm": True, "qk_norm_eps": EPS})

            toy_position = PartSpec("toy_interpolated", {
                "rotary_dim": ROTARY, "theta": THETA, "scale": SCALE, "max_positions": POSITIONS})
            rope = PartSpec("rope", {"head_dim": HEAD_DIM, "rotary_dim": HEAD_DIM, "theta": THETA, "max_positions": POSITIONS})
            routed = PartSpec("toy_routed", {"hidden_size": HIDDEN, "inner_size": INNER, "experts": EXPERTS})
            dense = PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": INNER})
            layers = (
                LayerSpec("prenorm", attention(toy_position), routed, norm, "model.layers.0."),
                LayerSpec("prenorm", attention(rope), dense, norm, "model.layers.1."),
                LayerSpec("prenorm", attention(toy_position), dense, norm, "model.layers.2."),
            )
            return ModelSpec(
                architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=HIDDEN, max_positions=POSITIONS,
                embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": HIDDEN}),
                layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(3)), final_norm=norm,
                head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": HIDDEN, "tied": False}),
            )

    register_architecture(ToyPartsConfig)
    return ToyPartsConfig


def plain_logits(weights, tokens):
    """The same model from the plain implementation's functions, whole sequence, no cache."""
    weights = {name: value.float() for name, value in weights.items()}
    positions = torch.arange(len(tokens))
    h = weights["model.embed_tokens.weight"][torch.as_tensor(tokens)]

    def attention(x, prefix, cos, sin):
        count = x.shape[0]
        q = (x @ weights[prefix + "q_proj.weight"].T).view(count, HEADS, HEAD_DIM)
        k = (x @ weights[prefix + "k_proj.weight"].T).view(count, KV_HEADS, HEAD_DIM)
        v = (x @ weights[prefix + "v_proj.weight"].T).view(count, KV_HEADS, HEAD_DIM)
        q = apply_rope(rms_norm(q, weights[prefix + "q_norm.weight"], EPS), cos, sin)
        k = apply_rope(rms_norm(k, weights[prefix + "k_norm.weight"], EPS), cos, sin)
        return causal_attention(q, k, v, HEAD_DIM**-0.5).reshape(count, -1) @ weights[prefix + "o_proj.weight"].T

    def routed(x, prefix):
        probability, expert = torch.softmax(x @ weights[prefix + "router.weight"].T, dim=-1).max(dim=-1)
        out = torch.zeros_like(x)
        for row in range(x.shape[0]):
            e = int(expert[row])
            hidden = torch.relu(x[row] @ weights[f"{prefix}experts.{e}.up.weight"].T)
            out[row] = probability[row] * (hidden @ weights[f"{prefix}experts.{e}.down.weight"].T)
        return out

    toy_angles = rope_angles(positions / SCALE, ROTARY, THETA)
    stock_angles = rope_angles(positions, HEAD_DIM, THETA)
    for index, (angles, feed_forward) in enumerate([(toy_angles, routed), (stock_angles, None), (toy_angles, None)]):
        prefix = f"model.layers.{index}."
        h = h + attention(rms_norm(h, weights[prefix + "input_layernorm.weight"], EPS), prefix + "self_attn.", *angles)
        x = rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], EPS)
        h = h + (routed(x, prefix + "mlp.") if feed_forward else swiglu(x, weights, prefix))
    return rms_norm(h, weights["model.norm.weight"], EPS) @ weights["lm_head.weight"].T


def test_a_routed_feed_forward_and_a_position_encoding_of_the_tests_own(tmp_path):
    from plain_qwen3 import read_safetensors

    from rapid_llm_b200.config import EngineConfig
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    config_class = register_toys()
    folder = write_random_model(tmp_path / "toy_parts", config_class(), seed=5)
    weights = read_safetensors(folder / "model.safetensors")
    assert "model.layers.0.mlp.experts.2.down.weight" in weights and "model.layers.1.mlp.gate_proj.weight" in weights
    engine = EngineConfig(dtype=torch.float32, max_seq_len=POSITIONS, page_size=8, num_pages=30, max_num_seqs=3,
                          max_num_batched_tokens=96, use_cuda_graph=False)
    runner = ModelRunner.from_folder(folder, engine)

    generator = torch.Generator().manual_seed(2)
    tokens = {name: torch.randint(0, VOCAB, (count,), generator=generator).tolist() for name, count in (("a", 70), ("b", 37))}
    plain = {name: plain_logits(weights, ids) for name, ids in tokens.items()}
    assert plain["a"].abs().max() > 0

    for name, ids in tokens.items():            # whole
        runner.admit(name)
        got = runner.step([StepEntry(name, ids, list(range(len(ids))))]).float().cpu()
        torch.testing.assert_close(got, plain[name], **for_dtype("float32"))
        runner.release(name)

    # portions of one beside single tokens of the other, in slots and pages that were used before
    for name in tokens:
        runner.admit(name)
    rows = {"a": [], "b": []}
    fed = {"a": 0, "b": 0}
    plan = [{"a": 9, "b": 30}, {"a": 2, "b": 1}, {"a": 33, "b": 1}, {"a": 1, "b": 1}, {"a": 25, "b": 4}]
    for sizes in plan:
        entries = []
        for name, size in sizes.items():
            entries.append(StepEntry(name, tokens[name][fed[name] : fed[name] + size], list(range(size))))
            fed[name] += size
        logits = runner.step(entries).float().cpu()
        at = 0
        for entry in entries:
            rows[entry.request_id].append(logits[at : at + len(entry.tokens)].clone())
            at += len(entry.tokens)
    runner.check_fault()
    for name in tokens:
        assert fed[name] == len(tokens[name])
        torch.testing.assert_close(torch.cat(rows[name]), plain[name], **for_dtype("float32"))
