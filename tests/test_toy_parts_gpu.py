"""Toy parts of the other roles, defined here and nowhere in the framework: a feed-forward that routes
each token to one of a few experts, a position encoding that is not the rotary one the framework ships, an
embedding that adds a learned row per absolute position; and, in a second model, a norm with a mean and a bias,
an arrangement that runs a layer's mixer and feed-forward side by side, and an output head that caps its logits.  They are registered, written as a
random model folder, loaded, and stepped whole, in portions and token by token through captured graphs, beside
the framework's own parts in other layers (different feed-forwards, windows, position encodings, norms and
arrangements layer by layer), in both precisions, against plain computations that are written out below.

The toys are arithmetic for a test, not a model of anyone's.
"""

from __future__ import annotations

import dataclasses

import pytest
import torch
from plain_qwen3 import apply_rope, causal_attention, load_model_dir, rms_norm, rope_angles, swiglu
from tolerances import at_scale

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, POSITIONS = 48, 211, 96
HEADS, KV_HEADS, HEAD_DIM, ROTARY = 6, 2, 32, 16
EPS, THETA, SLOW = 3e-6, 5000.0, 2.5
WINDOW = 8
EXPERTS = (3, 0, 2)          # experts of the routed feed-forward per layer; 0 = the framework's dense one
INNER = 40
SAFE_MARGIN = 0.05           # smallest gap between the two best router logits that the test's sequences keep


def toy_angles(positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The toy position encoding: frequencies 1 / (1 + i), positions slowed by a constant."""
    inv_freq = 1.0 / (1.0 + torch.arange(ROTARY // 2, dtype=torch.float32))
    angles = (positions.to(torch.float32) / SLOW)[:, None] * inv_freq[None, :]
    return torch.cos(angles), torch.sin(angles)


def register_toys():
    from rapid_llm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from rapid_llm_b200.ops import kernels
    from rapid_llm_b200.parts import TensorSpec
    from rapid_llm_b200.parts.base import EMBEDDINGS, FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, Part, PositionEncoding

    @POSITION_ENCODINGS.register("toy_slowed_rotation")
    class ToySlowedRotation(PositionEncoding):
        def __init__(self, *, rotary_dim, max_positions, dtype, device):
            super().__init__(dtype=dtype, device=device)
            assert rotary_dim == ROTARY
            cos, sin = toy_angles(torch.arange(max_positions))
            self.cos, self.sin = cos.to(device).contiguous(), sin.to(device).contiguous()

        def tables(self):
            return self.cos, self.sin

    @EMBEDDINGS.register("toy_token_plus_position")
    class ToyTokenPlusPosition(Part):
        """x_t = E[id_t] + P[position_t]."""

        def __init__(self, *, vocab_size, hidden_size, max_positions, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.weight = self.new_storage((vocab_size, hidden_size), "matrix")
            self.places = self.new_storage((max_positions, hidden_size), "matrix")

        def tensor_specs(self):
            return {"weight": TensorSpec(tuple(self.weight.shape)), "places": TensorSpec(tuple(self.places.shape))}

        def load_tensor(self, name, tensor):
            {"weight": self.weight, "places": self.places}[name].copy_(tensor)

        def forward(self, batch):
            out = batch.workspace.get("embedded", batch.num_tokens, self.weight.shape[1], self.dtype)
            kernels.embedding(out, self.weight, batch.token_ids, batch.fault, batch.feedback)
            summed = out.float() + self.places[batch.positions.long()].float()      # device indices: capturable
            return out.copy_(summed.to(self.dtype))

    @FEED_FORWARDS.register("toy_one_of_experts")
    class ToyOneOfExperts(FeedForward):
        """Router logits in float32, the best expert alone runs for a token, its result times its softmax weight.
        Every expert is computed for every token and masked: no shape depends on the routing, so a decode
        step can be captured."""

        def __init__(self, *, hidden_size, inner_size, experts, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.router = self.new_storage((experts, hidden_size), "vector")      # kept in float32
            self.up = self.new_storage((experts, inner_size, hidden_size), "matrix")
            self.down = self.new_storage((experts, hidden_size, inner_size), "matrix")

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec(tuple(self.router.shape), "vector")}
            for expert in range(self.up.shape[0]):
                specs[f"experts.{expert}.up.weight"] = TensorSpec(tuple(self.up.shape[1:]))
                specs[f"experts.{expert}.down.weight"] = TensorSpec(tuple(self.down.shape[1:]))
            return specs

        def load_tensor(self, name, tensor):
            if name == "router.weight":
                self.router.copy_(tensor.to(torch.float32))
                return
            _, expert, which, _ = name.split(".")
            (self.up if which == "up" else self.down)[int(expert)].copy_(tensor)

        def forward(self, x, batch):
            logits = x.float() @ self.router.T
            share = torch.softmax(logits, dim=-1)
            best = logits.argmax(dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for expert in range(self.up.shape[0]):
                inner = torch.relu(x @ self.up[expert].T)
                result = (inner @ self.down[expert].T).float()
                out += result * (share[:, expert] * (best == expert))[:, None]
            return out.to(x.dtype)

    @dataclasses.dataclass(frozen=True)
    class ToyPartsConfig:
        vocab_size: int
        architecture = "ToyPartsForCausalLM"
        model_type = "toy_parts"

        @classmethod
        def from_dict(cls, raw, overrides=None):
            return cls(dict(raw, **(overrides or {}))["vocab_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": self.model_type, "vocab_size": self.vocab_size}

        def to_spec(self):
            norm = PartSpec("rmsnorm", {"size": HIDDEN, "eps": EPS})
            toy_position = PartSpec("toy_slowed_rotation", {"rotary_dim": ROTARY, "max_positions": POSITIONS})
            rope = PartSpec("rope", {"head_dim": HEAD_DIM, "rotary_dim": ROTARY, "theta": THETA, "max_positions": POSITIONS})
            layers = []
            for index, experts in enumerate(EXPERTS):
                attention = PartSpec("gqa_attention", {
                    "hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
                    "position": rope if index == 1 else toy_position, "qk_norm": index != 2, "qk_norm_eps": EPS,
                    "window": WINDOW if index == 1 else 0,
                })
                if experts:
                    ffn = PartSpec("toy_one_of_experts", {"hidden_size": HIDDEN, "inner_size": INNER, "experts": experts})
                else:
                    ffn = PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": 2 * INNER})
                layers.append(LayerSpec("prenorm", attention, ffn, norm, f"model.layers.{index}."))
            return ModelSpec(
                architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=HIDDEN, max_positions=POSITIONS,
                embedding=PartSpec("toy_token_plus_position",
                                   {"vocab_size": self.vocab_size, "hidden_size": HIDDEN, "max_positions": POSITIONS}),
                layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm,
                head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": HIDDEN, "tied": True}),
            )

    register_architecture(ToyPartsConfig)
    return ToyPartsConfig


@torch.no_grad()
def plain_logits(weights: dict, ids: list[int]) -> tuple[torch.Tensor, float]:
    """Logits of one whole sequence in float32, and the smallest gap between the two best router logits."""
    positions = torch.arange(len(ids))
    h = weights["model.embed_tokens.weight"][ids] + weights["model.embed_tokens.places"][positions]
    smallest = float("inf")
    for index, experts in enumerate(EXPERTS):
        prefix = f"model.layers.{index}."
        x = rms_norm(h, weights[prefix + "input_layernorm.weight"], EPS)
        tokens = x.shape[0]
        q = (x @ weights[prefix + "self_attn.q_proj.weight"].T).view(tokens, HEADS, HEAD_DIM)
        k = (x @ weights[prefix + "self_attn.k_proj.weight"].T).view(tokens, KV_HEADS, HEAD_DIM)
        v = (x @ weights[prefix + "self_attn.v_proj.weight"].T).view(tokens, KV_HEADS, HEAD_DIM)
        if index != 2:
            q = rms_norm(q, weights[prefix + "self_attn.q_norm.weight"], EPS)
            k = rms_norm(k, weights[prefix + "self_attn.k_norm.weight"], EPS)
        cos, sin = rope_angles(positions, ROTARY, THETA) if index == 1 else toy_angles(positions)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        attended = causal_attention(q, k, v, HEAD_DIM**-0.5, WINDOW if index == 1 else 0)
        h = h + attended.reshape(tokens, HEADS * HEAD_DIM) @ weights[prefix + "self_attn.o_proj.weight"].T
        x = rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], EPS)
        if not experts:
            h = h + swiglu(x, weights, prefix)
            continue
        logits = x @ weights[prefix + "mlp.router.weight"].T
        top = logits.topk(2, dim=-1).values
        smallest = min(smallest, float((top[:, 0] - top[:, 1]).min()))
        share, best = torch.softmax(logits, dim=-1), logits.argmax(dim=-1)
        out = torch.zeros_like(h)
        for token in range(tokens):
            expert = int(best[token])
            inner = torch.relu(x[token] @ weights[prefix + f"mlp.experts.{expert}.up.weight"].T)
            out[token] = share[token, expert] * (inner @ weights[prefix + f"mlp.experts.{expert}.down.weight"].T)
        h = h + out
    h = rms_norm(h, weights["model.norm.weight"], EPS)
    return h @ weights["model.embed_tokens.weight"].T, smallest


def sequences_with_clear_routing(weights, lengths, seed):
    """Token sequences whose router decisions are not near a tie: a rounding error must not be able to send a
    token to another expert, or the comparison would test the luck of the draw."""
    generator = torch.Generator().manual_seed(seed)
    chosen = {}
    for name, length in lengths.items():
        for _ in range(2000):
            ids = torch.randint(0, VOCAB, (length,), generator=generator).tolist()
            logits, margin = plain_logits(weights, ids)
            if margin > SAFE_MARGIN:
                chosen[name] = (ids, logits)
                break
        else:
            raise AssertionError(f"no sequence of {length} tokens with router margins above {SAFE_MARGIN}")
    return chosen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routing_feed_forward_position_encoding_and_embedding(tmp_path, dtype):
    from rapid_llm_b200.config import EngineConfig
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    config_class = register_toys()
    torch_dtype = getattr(torch, dtype)
    folder = write_random_model(tmp_path / "toy_parts", config_class(VOCAB), seed=21, dtype=torch_dtype, std=0.12, norm_std=0.2)
    _, weights = load_model_dir(folder)
    assert "model.layers.0.mlp.router.weight" in weights and "model.layers.1.mlp.gate_proj.weight" in weights
    assert "model.layers.2.self_attn.q_norm.weight" not in weights and "model.embed_tokens.places" in weights

    engine = EngineConfig(dtype=torch_dtype, max_seq_len=POSITIONS, page_size=8, num_pages=40, max_num_seqs=3,
                          max_num_batched_tokens=96, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    kinds = [(type(layer.feed_forward).__name__, layer.mixer.window) for layer in runner.model.layers]
    assert kinds == [("ToyOneOfExperts", 0), ("SwiGLU", WINDOW), ("ToyOneOfExperts", 0)]
    assert len(runner.cache.groups) == 2          # all keys for two layers, a window of them for one

    tail = 9
    plain = sequences_with_clear_routing(weights, {"a": 33, "b": 20, "c": 27}, seed=5)

    # each request alone and whole
    for name, (ids, want) in plain.items():
        runner.admit(name)
        got = runner.step([StepEntry(name, ids, list(range(len(ids))))]).float().cpu()
        runner.release(name)
        torch.testing.assert_close(got, want, **at_scale(dtype, want))
        assert float(want.abs().max()) > 0.05

    # in portions side by side, then the last tokens one by one from captured graphs
    cuts = {"a": [5, 2, 17], "b": [9, 2], "c": [2, 13, 3]}
    fed = {name: 0 for name in plain}
    pieces = {name: [] for name in plain}
    for name in plain:
        runner.admit(name)
    for step in range(3):
        entries = []
        for name, (ids, _) in plain.items():
            if step < len(cuts[name]):
                size = cuts[name][step]
                entries.append(StepEntry(name, ids[fed[name] : fed[name] + size], list(range(size))))
                fed[name] += size
        logits = runner.step(entries).float().cpu()
        at = 0
        for entry in entries:
            pieces[entry.request_id].append(logits[at : at + len(entry.tokens)].clone())
            at += len(entry.tokens)
    while any(fed[name] < len(ids) for name, (ids, _) in plain.items()):
        live = [name for name, (ids, _) in plain.items() if fed[name] < len(ids)]
        entries = [StepEntry(name, [plain[name][0][fed[name]]], [0]) for name in live]
        logits = runner.step_decode(entries).float().cpu()
        for row, name in enumerate(live):
            pieces[name].append(logits[row : row + 1].clone())
            fed[name] += 1
    runner.check_fault()
    assert runner._graphs, "the decode steps were not captured"
    for name, (ids, want) in plain.items():
        torch.testing.assert_close(torch.cat(pieces[name]), want, **at_scale(dtype, want))
        assert sum(cuts[name]) + tail <= len(ids)


# ---------------------------------------------------------------------------------------------------
# The two remaining roles: a norm and an arrangement of a layer's parts, again defined here alone.
LN_EPS = 2e-5
HEAD_CAP = 1.5


def register_norm_and_arrangement():
    from rapid_llm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from rapid_llm_b200.parts import TensorSpec
    from rapid_llm_b200.parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Norm, Part
    from rapid_llm_b200.parts.base import HEADS as OUTPUT_HEADS
    from rapid_llm_b200.parts.norm import ADD, FIRST

    @OUTPUT_HEADS.register("toy_capped_head")
    class ToyCappedHead(Part):
        """logits = cap * tanh((h W^T) / cap): an output head of the test's own (its product is the framework's)."""

        def __init__(self, *, vocab_size, hidden_size, cap, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.cap = cap
            self.weight = self.new_storage((vocab_size, hidden_size), "matrix")

        def tensor_specs(self):
            return {"weight": TensorSpec(tuple(self.weight.shape))}

        def load_tensor(self, name, tensor):
            self.weight.copy_(tensor)

        def forward(self, hidden_rows, batch):
            from rapid_llm_b200.ops import gemm

            out = batch.workspace.get("logits", hidden_rows.shape[0], self.weight.shape[0], hidden_rows.dtype, min_rows=64)
            gemm.linear(hidden_rows, self.weight, out, batch.fault)
            gemm.flush()
            return out.copy_((self.cap * torch.tanh(out.float() / self.cap)).to(out.dtype))

    @NORMS.register("toy_layernorm")
    class ToyLayerNorm(Norm):
        """y = (r - mean(r)) / sqrt(var(r) + eps) * w + b with r = x or x + residual: a norm with a bias and a mean,
        which no product can take along (it makes no such offer and runs by itself, on torch's kernels)."""

        def __init__(self, *, size, eps, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.size, self.eps = size, eps
            self.weight = self.new_storage((size,), "vector")
            self.bias = self.new_storage((size,), "vector")

        def tensor_specs(self):
            return {"weight": TensorSpec((self.size,), "vector", init="ones_normal"), "bias": TensorSpec((self.size,), "vector")}

        def load_tensor(self, name, tensor):
            {"weight": self.weight, "bias": self.bias}[name].copy_(tensor.to(torch.float32))

        def forward(self, x, residual, batch, *, mode, write_residual, row_index=None, name="normed"):
            rows = x if row_index is None else x[row_index.long()]
            summed = rows.float()
            if mode == ADD:
                summed = summed + (residual if row_index is None else residual[row_index.long()])
            if write_residual:
                residual.copy_(summed)
            centred = summed - summed.mean(dim=-1, keepdim=True)
            out = centred * torch.rsqrt(centred.pow(2).mean(dim=-1, keepdim=True) + self.eps) * self.weight + self.bias
            return out.to(x.dtype)

    @BLOCKS.register("toy_parallel")
    class ToyParallelBlock(Block):
        """h' = h + Mixer(Norm(h)) + FeedForward(Norm(h)): one norm, both parts read it, both results join the
        residual stream.  The pair it hands on is (mixer's result + feed-forward's result, h)."""

        def __init__(self, *, layer, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.norm = NORMS.build(layer.norm, dtype=dtype, device=device)
            self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)
            self.children = (("only_norm.", self.norm), ("self_attn.", self.mixer), ("mlp.", self.feed_forward))

        def cache_need(self):
            return self.mixer.cache_need()

        def step_planners(self):
            planner = self.mixer.step_planner()
            return [] if planner is None else [planner]

        def tensor_specs(self):
            return {prefix + name: spec for prefix, part in self.children for name, spec in part.tensor_specs().items()}

        def load_tensor(self, name, tensor):
            for prefix, part in self.children:
                if name.startswith(prefix):
                    return part.load_tensor(name[len(prefix):], tensor)
            raise KeyError(name)

        def finalize(self, loaded):
            for prefix, part in self.children:
                part.finalize({name[len(prefix):] for name in loaded if name.startswith(prefix)})

        def forward(self, x, residual, batch, cache, then_norm=None):
            from rapid_llm_b200.ops import gemm

            gemm.flush()          # this block reads results with torch's kernels
            if residual is None:
                residual = batch.workspace.get("residual", x.shape[0], x.shape[1], torch.float32)
                normed = self.norm.forward(x, residual, batch, mode=FIRST, write_residual=True)
            else:
                normed = self.norm.forward(x, residual, batch, mode=ADD, write_residual=True)
            mixed = self.mixer.forward(normed, batch, cache)
            fed = self.feed_forward.forward(normed, batch)
            gemm.flush()
            both = batch.workspace.get("toy_both", x.shape[0], x.shape[1], x.dtype)
            both.copy_((mixed.float() + fed.float()).to(x.dtype))
            return both, residual

    @dataclasses.dataclass(frozen=True)
    class ToyArrangedConfig:
        vocab_size: int
        architecture = "ToyArrangedForCausalLM"
        model_type = "toy_arranged"

        @classmethod
        def from_dict(cls, raw, overrides=None):
            return cls(dict(raw, **(overrides or {}))["vocab_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": self.model_type, "vocab_size": self.vocab_size}

        def to_spec(self):
            layer_norm = PartSpec("toy_layernorm", {"size": HIDDEN, "eps": LN_EPS})
            rms = PartSpec("rmsnorm", {"size": HIDDEN, "eps": EPS})
            rope = PartSpec("rope", {"head_dim": HEAD_DIM, "rotary_dim": HEAD_DIM, "theta": THETA, "max_positions": POSITIONS})
            attention = PartSpec("gqa_attention", {"hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS,
                                                   "head_dim": HEAD_DIM, "position": rope, "qk_norm": True, "qk_norm_eps": EPS})
            ffn = PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": 2 * INNER})
            layers = (
                LayerSpec("prenorm", attention, ffn, layer_norm, "model.layers.0."),        # the stock arrangement, the toy norm
                LayerSpec("toy_parallel", attention, ffn, rms, "model.layers.1."),          # the toy arrangement, the stock norm
                LayerSpec("toy_parallel", attention, ffn, layer_norm, "model.layers.2."),   # both toys
                LayerSpec("prenorm", attention, ffn, rms, "model.layers.3."),               # all stock, after a toy block
            )
            return ModelSpec(
                architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=HIDDEN, max_positions=POSITIONS,
                embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": HIDDEN}),
                layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=layer_norm,
                head=PartSpec("toy_capped_head", {"vocab_size": self.vocab_size, "hidden_size": HIDDEN, "cap": HEAD_CAP}),
            )

    register_architecture(ToyArrangedConfig)
    return ToyArrangedConfig


@torch.no_grad()
def plain_arranged_logits(weights: dict, ids: list[int]) -> torch.Tensor:
    def layer_norm(h, prefix):
        centred = h - h.mean(dim=-1, keepdim=True)
        return centred * torch.rsqrt(centred.pow(2).mean(dim=-1, keepdim=True) + LN_EPS) * weights[prefix + "weight"] + weights[prefix + "bias"]

    def attention(x, prefix):
        tokens = x.shape[0]
        positions = torch.arange(tokens)
        q = rms_norm((x @ weights[prefix + "q_proj.weight"].T).view(tokens, HEADS, HEAD_DIM), weights[prefix + "q_norm.weight"], EPS)
        k = rms_norm((x @ weights[prefix + "k_proj.weight"].T).view(tokens, KV_HEADS, HEAD_DIM), weights[prefix + "k_norm.weight"], EPS)
        v = (x @ weights[prefix + "v_proj.weight"].T).view(tokens, KV_HEADS, HEAD_DIM)
        cos, sin = rope_angles(positions, HEAD_DIM, THETA)
        out = causal_attention(apply_rope(q, cos, sin), apply_rope(k, cos, sin), v, HEAD_DIM**-0.5)
        return out.reshape(tokens, HEADS * HEAD_DIM) @ weights[prefix + "o_proj.weight"].T

    h = weights["model.embed_tokens.weight"][ids]
    p = "model.layers.0."
    h = h + attention(layer_norm(h, p + "input_layernorm."), p + "self_attn.")
    h = h + swiglu(layer_norm(h, p + "post_attention_layernorm."), weights, p)
    p = "model.layers.1."
    x = rms_norm(h, weights[p + "only_norm.weight"], EPS)
    h = h + attention(x, p + "self_attn.") + swiglu(x, weights, p)
    p = "model.layers.2."
    x = layer_norm(h, p + "only_norm.")
    h = h + attention(x, p + "self_attn.") + swiglu(x, weights, p)
    p = "model.layers.3."
    h = h + attention(rms_norm(h, weights[p + "input_layernorm.weight"], EPS), p + "self_attn.")
    h = h + swiglu(rms_norm(h, weights[p + "post_attention_layernorm.weight"], EPS), weights, p)
    return HEAD_CAP * torch.tanh(layer_norm(h, "model.norm.") @ weights["lm_head.weight"].T / HEAD_CAP)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_norm_and_toy_arrangement(tmp_path, dtype):
    """A norm with a mean and a bias and a block that runs mixer and feed-forward side by side, in layers between
    stock blocks (so that norms ride on products in some layers and run by themselves in others): whole, in portions
    side by side, and token by token from captured graphs, against the plain computation above."""
    from rapid_llm_b200.config import EngineConfig
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.weights import write_random_model

    config_class = register_norm_and_arrangement()
    torch_dtype = getattr(torch, dtype)
    folder = write_random_model(tmp_path / "toy_arranged", config_class(VOCAB), seed=23, dtype=torch_dtype, std=0.1, norm_std=0.2)
    _, weights = load_model_dir(folder)
    assert "model.layers.1.only_norm.weight" in weights and "model.layers.2.only_norm.bias" in weights
    assert "model.layers.0.input_layernorm.bias" in weights and "model.norm.bias" in weights
    engine = EngineConfig(dtype=torch_dtype, max_seq_len=POSITIONS, page_size=8, num_pages=40, max_num_seqs=3,
                          max_num_batched_tokens=96, use_cuda_graph=True)
    runner = ModelRunner.from_folder(folder, engine)
    assert [type(layer).__name__ for layer in runner.model.layers] == ["PreNormBlock", "ToyParallelBlock", "ToyParallelBlock", "PreNormBlock"]

    generator = torch.Generator().manual_seed(6)
    tokens = {name: torch.randint(0, VOCAB, (count,), generator=generator).tolist() for name, count in (("a", 31), ("b", 18))}
    plain = {name: plain_arranged_logits(weights, ids) for name, ids in tokens.items()}
    for name, ids in tokens.items():
        runner.admit(name)
        got = runner.step([StepEntry(name, ids, list(range(len(ids))))]).float().cpu()
        runner.release(name)
        torch.testing.assert_close(got, plain[name], **at_scale(dtype, plain[name]))

    cuts, fed, pieces = {"a": [6, 2, 14], "b": [7, 3]}, {"a": 0, "b": 0}, {"a": [], "b": []}
    for name in tokens:
        runner.admit(name)
    for step in range(3):
        entries = []
        for name, ids in tokens.items():
            if step < len(cuts[name]):
                size = cuts[name][step]
                entries.append(StepEntry(name, ids[fed[name] : fed[name] + size], list(range(size))))
                fed[name] += size
        logits = runner.step(entries).float().cpu()
        at = 0
        for entry in entries:
            pieces[entry.request_id].append(logits[at : at + len(entry.tokens)].clone())
            at += len(entry.tokens)
    while any(fed[name] < len(ids) for name, ids in tokens.items()):
        live = [name for name, ids in tokens.items() if fed[name] < len(ids)]
        logits = runner.step_decode([StepEntry(name, [tokens[name][fed[name]]], [0]) for name in live]).float().cpu()
        for row, name in enumerate(live):
            pieces[name].append(logits[row : row + 1].clone())
            fed[name] += 1
    runner.check_fault()
    assert runner._graphs
    for name in tokens:
        torch.testing.assert_close(torch.cat(pieces[name]), plain[name], **at_scale(dtype, plain[name]))
