"""Each part alone on the GPU against the plain function of the same part, a run order
that names a layer twice and shares a cache, and a toy mixer with state of its own that is
registered, built and stepped without touching the framework's files."""

from __future__ import annotations

import dataclasses
import json

import pytest
import torch
from plain_qwen3 import attention_block, decoder_layer, geometry, rms_norm, rope_angles, swiglu
from tiny_configs import PAGE_SIZES
from tolerances import for_dtype

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def runner_for(folder, dtype, name, max_tokens=256):
    from rapid_llm_b200.config import load_config
    from rapid_llm_b200.engine.runner import ModelRunner
    from rapid_llm_b200.replay import engine_config_for

    return ModelRunner.from_folder(folder, engine_config_for(load_config(folder), dtype, max_tokens, PAGE_SIZES[name]))


def whole_batch(runner, count, request_id="p"):
    from rapid_llm_b200.engine.runner import StepEntry

    runner.admit(request_id)
    return runner.prepare([StepEntry(request_id, [1] * count, [])])


@pytest.fixture(scope="module")
def folders(tiny_dirs, tiny_dirs_bf16, tiny_plain, tiny_plain_bf16):
    return {"float32": (tiny_dirs, tiny_plain), "bfloat16": (tiny_dirs_bf16, tiny_plain_bf16)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_norm_feed_forward_attention_and_block(name, dtype, folders):
    dirs, plains = folders[dtype]
    config, weights = plains[name]
    cfg = geometry(config)
    runner = runner_for(dirs[name], dtype, name)
    tokens, hidden = 45, config["hidden_size"]
    batch = whole_batch(runner, tokens)
    caches = runner.layer_caches()
    layer = runner.model.layers[1]
    prefix = "model.layers.1."
    tol = for_dtype(dtype)
    x = torch.randn(tokens, hidden).to(runner.dtype)
    x_plain = x.float()
    x_dev = x.to(runner.device)

    from rapid_llm_b200.parts.norm import PLAIN

    normed = layer.mixer_norm.forward(x_dev, None, batch, mode=PLAIN, write_residual=False)
    torch.testing.assert_close(normed.float().cpu(), rms_norm(x_plain, weights[prefix + "input_layernorm.weight"], cfg["eps"]), **tol)

    out = layer.feed_forward.forward(x_dev, batch)
    torch.testing.assert_close(out.float().cpu(), swiglu(x_plain, weights, prefix), **tol)

    windows = [spec.mixer.params["window"] for spec in runner.model.spec.layers]
    out = layer.mixer.forward(x_dev, batch, caches[1])
    want = attention_block(x_plain, weights, prefix, cfg, torch.arange(tokens), windows[1])
    torch.testing.assert_close(out.float().cpu(), want, **tol)

    y, residual = layer.forward(x_dev, None, batch, caches[1])
    want = decoder_layer(x_plain, weights, prefix, cfg, torch.arange(tokens), windows[1])
    torch.testing.assert_close((y.float() + residual).cpu(), want, **tol)
    runner.check_fault()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens", [23, 150])      # a step of the streaming product; one of the library product
def test_attention_with_a_bias_on_q_k_and_v(dtype, tokens, folders):
    """The attention part built with ``qkv_bias`` (no model here has one): its checkpoint names, and the
    bias added in float32 before the per-head norms, against the plain functions put together by hand."""
    from plain_qwen3 import apply_rope, causal_attention
    from rapid_llm_b200.config import PartSpec
    from rapid_llm_b200.parts import MIXERS

    hidden, heads, kv_heads, dim, eps, theta = 80, 6, 3, 48, 3e-6, 50000.0
    part = MIXERS.build(PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": dim, "qk_norm": True,
        "qk_norm_eps": eps, "qkv_bias": True,
        "position": PartSpec("rope", {"head_dim": dim, "rotary_dim": dim, "theta": theta, "max_positions": 512}),
    }), dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], device="cuda:0")
    specs = part.tensor_specs()
    assert {"q_proj.bias", "k_proj.bias", "v_proj.bias"} <= set(specs) and specs["k_proj.bias"].shape == (kv_heads * dim,)
    generator = torch.Generator().manual_seed(12)
    weights = {}
    for name, spec in specs.items():
        scale = 0.5 if name.endswith("bias") else 0.05
        value = torch.randn(spec.shape, generator=generator) * scale + (1.0 if "norm" in name else 0.0)
        weights[name] = value.to(part.dtype).float() if spec.kind == "matrix" else value
        part.load_tensor(name, weights[name])

    dirs, _ = folders[dtype]
    runner = runner_for(dirs["C"], dtype, "C")           # a cache of the same geometry (3 kv heads of 48)
    batch = whole_batch(runner, tokens)
    x = torch.randn(tokens, hidden, generator=generator).to(part.dtype)
    out = part.forward(x.to("cuda:0"), batch, runner.layer_caches()[0])
    runner.check_fault()

    xf = x.float()
    q = (xf @ weights["q_proj.weight"].T + weights["q_proj.bias"]).view(tokens, heads, dim)
    key = (xf @ weights["k_proj.weight"].T + weights["k_proj.bias"]).view(tokens, kv_heads, dim)
    value = (xf @ weights["v_proj.weight"].T + weights["v_proj.bias"]).view(tokens, kv_heads, dim)
    q, key = rms_norm(q, weights["q_norm.weight"], eps), rms_norm(key, weights["k_norm.weight"], eps)
    cos, sin = rope_angles(torch.arange(tokens), dim, theta)
    attended = causal_attention(apply_rope(q, cos, sin), apply_rope(key, cos, sin), value, dim**-0.5)
    want = attended.reshape(tokens, heads * dim) @ weights["o_proj.weight"].T
    torch.testing.assert_close(out.float().cpu(), want, **for_dtype(dtype))


def test_rope_tables_are_the_plain_angles():
    from rapid_llm_b200.parts.rope import RotaryEmbedding

    part = RotaryEmbedding(head_dim=48, rotary_dim=32, theta=50000.0, max_positions=300, dtype=torch.float32, device="cuda:0")
    cos, sin = part.tables()
    want_cos, want_sin = rope_angles(torch.arange(300), 32, 50000.0)
    assert torch.equal(cos.cpu(), want_cos) and torch.equal(sin.cpu(), want_sin)
    again = RotaryEmbedding(head_dim=48, rotary_dim=32, theta=50000.0, max_positions=300, dtype=torch.float32, device="cuda:0")
    assert again.tables()[0] is cos, "layers with the same encoding share one table"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head(dtype, folders):
    dirs, plains = folders[dtype]
    config, weights = plains["B"]
    runner = runner_for(dirs["B"], dtype, "B")
    from rapid_llm_b200.engine.runner import StepEntry

    runner.admit("e")
    ids = torch.randint(0, config["vocab_size"], (19,)).tolist()
    batch = runner.prepare([StepEntry("e", ids, [])])
    embedded = runner.model.embedding.forward(batch)
    assert torch.equal(embedded.float().cpu(), weights["model.embed_tokens.weight"][ids].to(runner.dtype).float())
    h = torch.randn(5, config["hidden_size"]).to(runner.dtype)
    logits = runner.model.head.forward(h.to(runner.device), batch)
    torch.testing.assert_close(logits.float().cpu(), h.float() @ weights["lm_head.weight"].T, **for_dtype(dtype))


def test_run_order_names_a_layer_twice(tmp_path, tiny_dirs, tiny_plain):
    """Run order [0, 1, 0]: layer 0 runs twice with its own cache each time."""
    from rapid_llm_b200.config import EngineConfig, ScheduleEntry, load_config
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.models import CausalLM
    from rapid_llm_b200.weights import load_weights

    config, weights = tiny_plain["A"]
    cfg = geometry(config)
    spec = load_config(tiny_dirs["A"]).to_spec()
    spec = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)))
    model = CausalLM(spec, torch.float32, "cuda:0")
    load_weights(model, tiny_dirs["A"])
    runner = ModelRunner(model, EngineConfig(dtype=torch.float32, max_seq_len=128, num_pages=16, max_num_seqs=2,
                                             max_num_batched_tokens=128, use_cuda_graph=False))
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].entries == (0, 1, 2)
    tokens = torch.randint(0, 256, (40,)).tolist()
    runner.admit("r")
    first = runner.step([StepEntry("r", tokens[:23], list(range(23)))]).clone()   # valid until the next step
    second = runner.step([StepEntry("r", tokens[23:], list(range(17)))])
    got = torch.cat([first, second]).cpu()
    h = weights["model.embed_tokens.weight"][tokens]
    positions = torch.arange(40)
    for index in (0, 1, 0):
        h = decoder_layer(h, weights, f"model.layers.{index}.", cfg, positions, 0)
    want = rms_norm(h, weights["model.norm.weight"], cfg["eps"]) @ weights["model.embed_tokens.weight"].T
    torch.testing.assert_close(got, want, **for_dtype("float32"))


# ------------------------------------------------------------------ a toy mixer
def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from rapid_llm_b200.config import EngineConfig, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.parts import MIXERS, Mixer, StateNeed, TensorSpec
    from rapid_llm_b200.weights import write_random_model

    @MIXERS.register("toy_decay")
    class ToyDecay(Mixer):
        """s_t = decay * s_{t-1} + x_t per request; y_t = s_t @ W^T.  Keeps s as per-request state."""

        def __init__(self, *, hidden_size, decay, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.hidden, self.decay = hidden_size, decay
            self.weight = self.new_storage((hidden_size, hidden_size), "matrix")

        def state_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def tensor_specs(self):
            return {"proj.weight": TensorSpec((self.hidden, self.hidden))}

        def load_tensor(self, name, tensor):
            assert name == "proj.weight"
            self.weight.copy_(tensor)

        def forward(self, x, batch, cache):
            out = torch.empty_like(x)
            for index in range(batch.num_entries):
                begin, end = int(batch.h_cu_seqlens[index]), int(batch.h_cu_seqlens[index + 1])
                slot = int(batch.h_entry_slot[index])
                state = cache.state[slot]
                for row in range(begin, end):
                    state.mul_(self.decay).add_(x[row].float())
                    out[row] = (state @ self.weight.float().T).to(x.dtype)
            return out

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        decay: float
        architecture = "ToyDecayForCausalLM"
        model_type = "toy_decay"

        @classmethod
        def from_dict(cls, raw, overrides=None):
            raw = dict(raw, **(overrides or {}))
            return cls(raw["vocab_size"], raw["hidden_size"], raw["decay"])

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": self.model_type, **dataclasses.asdict(self)}

        def to_spec(self):
            norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": 1e-5})
            toy = PartSpec("toy_decay", {"hidden_size": self.hidden_size, "decay": self.decay})
            attention = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                "position": PartSpec("rope", {"head_dim": 16, "rotary_dim": 16, "theta": 10000.0, "max_positions": 64}),
            })
            ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": 2 * self.hidden_size})
            layers = tuple(
                LayerSpec("prenorm", mixer, ffn, norm, f"model.layers.{i}.") for i, mixer in enumerate((toy, attention, toy))
            )
            return ModelSpec(
                architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size, max_positions=64,
                embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
                layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(3)), final_norm=norm,
                head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": True}),
            )

    register_architecture(ToyConfig)
    folder = write_random_model(tmp_path / "toy", ToyConfig(97, 32, 0.5), seed=3)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyDecayForCausalLM"]
    engine = EngineConfig(dtype=torch.float32, max_seq_len=64, page_size=8, num_pages=16, max_num_seqs=3,
                          max_num_batched_tokens=64, use_cuda_graph=False)
    runner = ModelRunner.from_folder(folder, engine)
    assert [need is not None for need in runner.model.state_needs()] == [True, False, True]
    assert runner.storage.states[0].shape == (4, 32) and runner.storage.states[1] is None

    tokens = {"a": torch.randint(0, 97, (30,)).tolist(), "b": torch.randint(0, 97, (21,)).tolist()}
    whole = {}
    for name, ids in tokens.items():
        runner.admit(name)
        whole[name] = runner.step([StepEntry(name, ids, list(range(len(ids))))]).cpu().clone()
        runner.release(name)
    # the same requests in portions, side by side, in slots that were used before
    for name in tokens:
        runner.admit(name)
    pieces = {"a": [], "b": []}
    cuts = {"a": [7, 2, 11, 10], "b": [1, 13, 7]}
    fed = {"a": 0, "b": 0}
    for step in range(4):
        entries = []
        for name in ("a", "b"):
            if step < len(cuts[name]):
                size = cuts[name][step]
                entries.append(StepEntry(name, tokens[name][fed[name] : fed[name] + size], list(range(size))))
                fed[name] += size
        logits = runner.step(entries).cpu()
        at = 0
        for entry in entries:
            pieces[entry.request_id].append(logits[at : at + len(entry.tokens)].clone())
            at += len(entry.tokens)
    for name in tokens:
        torch.testing.assert_close(torch.cat(pieces[name]), whole[name], **for_dtype("float32"))
    assert float(whole["a"].abs().max()) > 0


def test_a_toy_mixer_with_rows_of_its_own_in_the_pages(tmp_path):
    """A mixer that caches one row per token of a width it chooses (neither keys nor values): the cache
    manager gives it pages ``[page, width]`` from its ``CacheNeed.token_shape``, in a group of its own beside the
    attention layer's, and the pages are used again by later requests.  y_t = mean of the rows 0..t, times W."""
    from rapid_llm_b200.config import EngineConfig, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.parts import MIXERS, CacheNeed, Mixer, TensorSpec
    from rapid_llm_b200.weights import write_random_model

    hidden, width, vocab = 32, 24, 83

    @MIXERS.register("toy_mean_of_rows")
    class ToyMeanOfRows(Mixer):
        def __init__(self, *, hidden_size, width, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.down = self.new_storage((width, hidden_size), "matrix")
            self.up = self.new_storage((hidden_size, width), "matrix")

        def cache_need(self):
            return CacheNeed("full", token_shape=(self.down.shape[0],))

        def tensor_specs(self):
            return {"down.weight": TensorSpec(tuple(self.down.shape)), "up.weight": TensorSpec(tuple(self.up.shape))}

        def load_tensor(self, name, tensor):
            (self.down if name == "down.weight" else self.up).copy_(tensor)

        def forward(self, x, batch, cache):
            group = batch.groups[cache.group]
            rows = x.float() @ self.down.float().T
            flat = cache.pages.view(-1, self.down.shape[0])            # [pages * page_size, width]
            flat[group.kv_dest.long()] = rows.to(flat.dtype)
            out = torch.empty_like(x)
            for index in range(batch.num_entries):
                begin, end = int(batch.h_cu_seqlens[index]), int(batch.h_cu_seqlens[index + 1])
                start, slot = int(batch.h_entry_start[index]), int(batch.h_entry_slot[index])
                count = start + end - begin
                pages = group.block_table[slot, : -(-count // group.page_size)].long()
                held = cache.pages[pages].reshape(-1, self.down.shape[0])[:count].float()
                means = held.cumsum(0)[start:] / torch.arange(start + 1, count + 1, device=x.device)[:, None]
                out[begin:end] = (means @ self.up.float().T).to(x.dtype)
            return out

    @dataclasses.dataclass(frozen=True)
    class RowsConfig:
        vocab_size: int
        architecture = "ToyMeanOfRowsForCausalLM"
        model_type = "toy_mean_of_rows"

        @classmethod
        def from_dict(cls, raw, overrides=None):
            return cls(dict(raw, **(overrides or {}))["vocab_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": self.model_type, "vocab_size": self.vocab_size}

        def to_spec(self):
            norm = PartSpec("rmsnorm", {"size": hidden, "eps": 1e-5})
            toy = PartSpec("toy_mean_of_rows", {"hidden_size": hidden, "width": width})
            attention = PartSpec("gqa_attention", {
                "hidden_size": hidden, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                "position": PartSpec("rope", {"head_dim": 16, "rotary_dim": 16, "theta": 10000.0, "max_positions": 64}),
            })
            ffn = PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 48})
            layers = tuple(LayerSpec("prenorm", mixer, ffn, norm, f"model.layers.{i}.") for i, mixer in enumerate((toy, attention, toy)))
            return ModelSpec(
                architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=hidden, max_positions=64,
                embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": hidden}),
                layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(3)), final_norm=norm,
                head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": hidden, "tied": True}),
            )

    register_architecture(RowsConfig)
    folder = write_random_model(tmp_path / "rows", RowsConfig(vocab), seed=5)
    engine = EngineConfig(dtype=torch.float32, max_seq_len=64, page_size=8, num_pages=9, max_num_seqs=3,
                          max_num_batched_tokens=64, use_cuda_graph=False)
    runner = ModelRunner.from_folder(folder, engine)
    shapes = sorted(tuple(pages.shape) for pages in runner.storage.pages)
    assert shapes == [(1, 10, 2, 1, 8, 16), (2, 10, 8, width)]         # keys and values of one layer; rows of two

    generator = torch.Generator().manual_seed(6)
    tokens = {name: torch.randint(0, vocab, (count,), generator=generator).tolist()
              for name, count in (("a", 30), ("b", 21), ("c", 37))}
    whole = {}
    for name, ids in tokens.items():
        runner.admit(name)
        whole[name] = runner.step([StepEntry(name, ids, list(range(len(ids))))]).cpu().clone()
        runner.release(name)
    # two at a time in portions, the third once pages are free again: 9 pages of 8 hold 72 tokens
    pieces = {name: [] for name in tokens}
    fed = {name: 0 for name in tokens}
    cuts = {"a": [7, 2, 11, 10], "b": [1, 13, 7], "c": [20, 2, 15]}
    for names in (("a", "b"), ("c",)):
        for name in names:
            runner.admit(name)
        for step in range(4):
            entries = []
            for name in names:
                if step < len(cuts[name]):
                    size = cuts[name][step]
                    entries.append(StepEntry(name, tokens[name][fed[name] : fed[name] + size], list(range(size))))
                    fed[name] += size
            if not entries:
                continue
            logits = runner.step(entries).cpu()
            at = 0
            for entry in entries:
                pieces[entry.request_id].append(logits[at : at + len(entry.tokens)].clone())
                at += len(entry.tokens)
        for name in names:
            runner.release(name)
        runner.cache.check()
    for name in tokens:
        torch.testing.assert_close(torch.cat(pieces[name]), whole[name], **for_dtype("float32"))


def test_state_advances_once_per_token_when_decode_steps_are_captured(tmp_path):
    """A mixer with state, indexed on the device, decodes through captured graphs: the step in
    which a batch size is captured must advance the state once, like every other step."""
    from rapid_llm_b200.config import EngineConfig, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from rapid_llm_b200.engine.runner import ModelRunner, StepEntry
    from rapid_llm_b200.parts import MIXERS, Mixer, StateNeed, TensorSpec
    from rapid_llm_b200.weights import write_random_model

    hidden, vocab, decay = 32, 89, 0.75

    @MIXERS.register("toy_running_sum")
    class ToyRunningSum(Mixer):
        """s_t = decay * s_{t-1} + x_t per request; y_t = s_t @ W^T."""

        def __init__(self, *, hidden_size, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.weight = self.new_storage((hidden_size, hidden_size), "matrix")

        def state_need(self):
            return StateNeed((self.weight.shape[0],), torch.float32)

        def tensor_specs(self):
            return {"proj.weight": TensorSpec(tuple(self.weight.shape))}

        def load_tensor(self, name, tensor):
            self.weight.copy_(tensor)

        def forward(self, x, batch, cache):
            if batch.decode_only:          # one token per entry: slots come from the device, no host decision
                slots = batch.entry_slot.long()
                state = cache.state[slots] * decay + x.float()
                cache.state[slots] = state
                return (state @ self.weight.float().T).to(x.dtype)
            out = torch.empty_like(x)
            for index in range(batch.num_entries):
                state = cache.state[int(batch.h_entry_slot[index])]
                for row in range(int(batch.h_cu_seqlens[index]), int(batch.h_cu_seqlens[index + 1])):
                    state.mul_(decay).add_(x[row].float())
                    out[row] = (state @ self.weight.float().T).to(x.dtype)
            return out

    @dataclasses.dataclass(frozen=True)
    class RunningSumConfig:
        vocab_size: int
        architecture = "ToyRunningSumForCausalLM"
        model_type = "toy_running_sum"

        @classmethod
        def from_dict(cls, raw, overrides=None):
            return cls(dict(raw, **(overrides or {}))["vocab_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": self.model_type, "vocab_size": self.vocab_size}

        def to_spec(self):
            norm = PartSpec("rmsnorm", {"size": hidden, "eps": 1e-5})
            toy = PartSpec("toy_running_sum", {"hidden_size": hidden})
            attention = PartSpec("gqa_attention", {
                "hidden_size": hidden, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                "position": PartSpec("rope", {"head_dim": 16, "rotary_dim": 16, "theta": 10000.0, "max_positions": 64}),
            })
            ffn = PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 48})
            layers = tuple(LayerSpec("prenorm", mixer, ffn, norm, f"model.layers.{i}.") for i, mixer in enumerate((toy, attention)))
            return ModelSpec(
                architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=hidden, max_positions=64,
                embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": hidden}),
                layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(2)), final_norm=norm,
                head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": hidden, "tied": True}),
            )

    register_architecture(RunningSumConfig)
    folder = write_random_model(tmp_path / "running_sum", RunningSumConfig(vocab), seed=11)
    engine = EngineConfig(dtype=torch.float32, max_seq_len=64, page_size=8, num_pages=24, max_num_seqs=4,
                          max_num_batched_tokens=64, use_cuda_graph=True, use_dependent_launch=False)
    runner = ModelRunner.from_folder(folder, engine)
    generator = torch.Generator().manual_seed(4)
    tokens = {name: torch.randint(0, vocab, (count,), generator=generator).tolist()
              for name, count in (("a", 19), ("b", 12), ("c", 26))}
    tail = 7
    whole = {}
    for name, ids in tokens.items():
        runner.admit(name)
        whole[name] = runner.step([StepEntry(name, ids, list(range(len(ids) - tail, len(ids))))]).cpu().clone()
        runner.release(name)

    for name, ids in tokens.items():
        runner.admit(name)
        runner.step([StepEntry(name, ids[:-tail], [])])
    decoded = {name: [] for name in tokens}
    for step in range(tail):        # three rows padded to a batch of four; the first of these steps captures it
        entries = [StepEntry(name, [ids[len(ids) - tail + step]], [0]) for name, ids in tokens.items()]
        logits = runner.step_decode(entries).cpu()
        for row, name in enumerate(tokens):
            decoded[name].append(logits[row].clone())
    runner.check_fault()
    assert [bucket for bucket, _ in runner._graphs] == [4]
    for name in tokens:
        torch.testing.assert_close(torch.stack(decoded[name]), whole[name], **for_dtype("float32"))
