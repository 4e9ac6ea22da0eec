"""Weight loading by name, its one error, and the random-weights mode (no GPU)."""

import json

import pytest
import torch
from plain_qwen3 import load_model_dir
from tiny_configs import TINY_A, TINY_B

from rapid_llm_b200.config import Qwen3Config, load_config
from rapid_llm_b200.models import CausalLM
from rapid_llm_b200.weights import SafetensorsFile, WeightLoadError, load_weights, write_random_model, write_safetensors


def build(folder, dtype=torch.float32):
    model = CausalLM(load_config(folder).to_spec(), dtype, "cpu")
    load_weights(model, folder)
    return model


def rewrite(folder, out, change):
    tensors = {}
    with SafetensorsFile(folder / "model.safetensors") as handle:
        for name in handle.keys():
            tensors[name] = handle.tensor(name).clone()
    change(tensors)
    out.mkdir()
    (out / "config.json").write_text((folder / "config.json").read_text())
    write_safetensors(out / "model.safetensors", tensors)
    return out


def test_every_tensor_lands_where_it_belongs(tiny_dirs):
    folder = tiny_dirs["B"]
    model = build(folder)
    _, weights = load_model_dir(folder)
    config = load_config(folder)
    q_rows = config.num_attention_heads * config.head_dim
    kv_rows = config.num_key_value_heads * config.head_dim
    for index, layer in enumerate(model.layers):
        prefix = f"model.layers.{index}."
        assert torch.equal(layer.mixer.qkv[:q_rows], weights[prefix + "self_attn.q_proj.weight"])
        assert torch.equal(layer.mixer.qkv[q_rows : q_rows + kv_rows], weights[prefix + "self_attn.k_proj.weight"])
        assert torch.equal(layer.mixer.qkv[q_rows + kv_rows :], weights[prefix + "self_attn.v_proj.weight"])
        assert torch.equal(layer.mixer.o, weights[prefix + "self_attn.o_proj.weight"])
        assert torch.equal(layer.mixer.q_norm, weights[prefix + "self_attn.q_norm.weight"])
        assert torch.equal(layer.mixer.k_norm, weights[prefix + "self_attn.k_norm.weight"])
        inter = config.intermediate_size
        assert torch.equal(layer.feed_forward.gate_up[:inter], weights[prefix + "mlp.gate_proj.weight"])
        assert torch.equal(layer.feed_forward.gate_up[inter:], weights[prefix + "mlp.up_proj.weight"])
        assert torch.equal(layer.feed_forward.down, weights[prefix + "mlp.down_proj.weight"])
        assert torch.equal(layer.mixer_norm.weight, weights[prefix + "input_layernorm.weight"])
        assert torch.equal(layer.feed_forward_norm.weight, weights[prefix + "post_attention_layernorm.weight"])
    assert torch.equal(model.final_norm.weight, weights["model.norm.weight"])
    assert torch.equal(model.head.weight, weights["lm_head.weight"])
    assert model.head.weight is not model.embedding.weight


def test_a_model_in_several_shards_loads_like_one_file(tiny_dirs, tmp_path):
    """Shards are read in name order; q, k and v of one layer may lie in different files.  A tensor
    that two shards hold is reported, not silently taken from one of them."""
    folder = tiny_dirs["B"]
    tensors = {}
    with SafetensorsFile(folder / "model.safetensors") as handle:
        for name in handle.keys():
            tensors[name] = handle.tensor(name).clone()
    names = sorted(tensors)
    out = tmp_path / "sharded"
    out.mkdir()
    (out / "config.json").write_text((folder / "config.json").read_text())
    for index in range(3):
        part = {name: tensors[name] for name in names[index::3]}
        write_safetensors(out / f"model-{index + 1:05d}-of-00003.safetensors", part)
    whole, sharded = build(folder), build(out)
    for a, b in zip(whole.layers, sharded.layers):
        assert torch.equal(a.mixer.qkv, b.mixer.qkv) and torch.equal(a.mixer.o, b.mixer.o)
        assert torch.equal(a.mixer.q_norm, b.mixer.q_norm) and torch.equal(a.mixer.k_norm, b.mixer.k_norm)
        assert torch.equal(a.feed_forward.gate_up, b.feed_forward.gate_up)
        assert torch.equal(a.feed_forward.down, b.feed_forward.down)
        assert torch.equal(a.mixer_norm.weight, b.mixer_norm.weight)
        assert torch.equal(a.feed_forward_norm.weight, b.feed_forward_norm.weight)
    assert torch.equal(whole.embedding.weight, sharded.embedding.weight)
    assert torch.equal(whole.head.weight, sharded.head.weight)
    assert torch.equal(whole.final_norm.weight, sharded.final_norm.weight)
    write_safetensors(out / "model-00004-of-00003.safetensors", {names[0]: tensors[names[0]]})
    with pytest.raises(WeightLoadError) as caught:
        build(out)
    assert names[0] in str(caught.value)


def test_tied_head_is_the_embedding_and_a_shipped_head_wins(tiny_dirs, tmp_path):
    model = build(tiny_dirs["A"])
    assert model.head.weight is model.embedding.weight
    shipped = rewrite(tiny_dirs["A"], tmp_path / "shipped",
                      lambda t: t.update({"lm_head.weight": torch.full_like(t["model.embed_tokens.weight"], 0.5)}))
    model = build(shipped)
    assert model.head.weight is not model.embedding.weight and float(model.head.weight[0, 0]) == 0.5


def test_dtypes_matrices_follow_the_engine_vectors_stay_32_bit(tiny_dirs, tiny_dirs_bf16):
    model = build(tiny_dirs["A"], torch.bfloat16)
    assert model.layers[0].mixer.qkv.dtype == torch.bfloat16
    assert model.layers[0].mixer_norm.weight.dtype == torch.float32
    assert model.layers[0].mixer.q_norm.dtype == torch.float32
    with SafetensorsFile(tiny_dirs_bf16["A"] / "model.safetensors") as handle:
        assert handle.dtype("model.embed_tokens.weight") == torch.bfloat16
        assert handle.dtype("model.norm.weight") == torch.float32
    widened = build(tiny_dirs_bf16["A"], torch.float32)
    assert widened.layers[0].mixer.qkv.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tiny_dirs, tmp_path):
    def change(tensors):
        del tensors["model.layers.1.mlp.up_proj.weight"]
        del tensors["model.norm.weight"]
        tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(4)
        tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(7, 96)
        tensors["model.layers.9.mlp.up_proj.weight"] = torch.zeros(2, 2)     # beyond the layer count: ignored

    broken = rewrite(tiny_dirs["B"], tmp_path / "broken", change)
    with pytest.raises(WeightLoadError) as info:
        build(broken)
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert error.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (7, 96), (32, 96))]
    text = str(error)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "file has [7, 96], model expects [32, 96]"):
        assert needle in text


def test_missing_head_without_tie_is_an_error(tiny_dirs, tmp_path):
    broken = rewrite(tiny_dirs["B"], tmp_path / "nohead", lambda t: t.pop("lm_head.weight"))
    with pytest.raises(WeightLoadError, match="lm_head.weight"):
        build(broken)


def test_no_safetensors_and_truncated_file(tiny_dirs, tmp_path):
    empty = tmp_path / "empty"
    empty.mkdir()
    (empty / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="safetensors"):
        build(empty)
    cut = tmp_path / "cut"
    cut.mkdir()
    (cut / "config.json").write_text(json.dumps(TINY_A))
    blob = (tiny_dirs["A"] / "model.safetensors").read_bytes()
    (cut / "model.safetensors").write_bytes(blob[: len(blob) // 2])
    with pytest.raises(ValueError, match="outside the file"):
        build(cut)


def test_random_mode_is_seeded_and_scaled(tmp_path):
    config = Qwen3Config.from_dict(TINY_B)
    first = write_random_model(tmp_path / "a", config, 5)
    again = write_random_model(tmp_path / "b", config, 5)
    other = write_random_model(tmp_path / "c", config, 6)
    assert (first / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    assert (first / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()
    assert json.loads((first / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    _, weights = load_model_dir(first)
    assert abs(float(weights["model.embed_tokens.weight"].std()) - 0.02) < 0.002
    norm = weights["model.layers.0.input_layernorm.weight"]
    assert abs(float(norm.mean()) - 1.0) < 0.05 and 0.05 < float(norm.std()) < 0.15
    assert "lm_head.weight" in weights
    tied = write_random_model(tmp_path / "tied", Qwen3Config.from_dict(TINY_A), 0)
    assert "lm_head.weight" not in load_model_dir(tied)[1]
