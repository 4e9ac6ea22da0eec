"""Configuration and registry (no GPU)."""

import json

import pytest
from tiny_configs import CONFIGS, TINY_A, TINY_B, TINY_C

from rapid_llm_b200.config import Qwen3Config, load_config, resolve_architecture, supported_architectures
from rapid_llm_b200.config.registry import read_config_json


def test_keys_are_read_not_assumed():
    for raw in CONFIGS.values():
        config = Qwen3Config.from_dict(raw)
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta"):
            assert getattr(config, key) == raw[key]
        spec = config.to_spec()
        assert len(spec.layers) == raw["num_hidden_layers"]
        assert [entry.layer for entry in spec.schedule] == list(range(raw["num_hidden_layers"]))
        mixer = spec.layers[0].mixer.params
        assert mixer["num_heads"] == raw["num_attention_heads"] and mixer["head_dim"] == raw["head_dim"]
        assert mixer["scale"] == raw["head_dim"] ** -0.5 and mixer["qk_norm"] is True
        assert spec.layers[0].norm.params["eps"] == raw["rms_norm_eps"]
        assert spec.head.params["tied"] == raw["tie_word_embeddings"]


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "tie_word_embeddings")}
    config = Qwen3Config.from_dict(raw)
    assert config.num_key_value_heads == raw["num_attention_heads"]
    assert config.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert config.rope_theta == 10000.0 and config.tie_word_embeddings is False


def test_explicit_head_dim_wins():
    assert Qwen3Config.from_dict(TINY_B).head_dim == 32 != TINY_B["hidden_size"] // TINY_B["num_attention_heads"]


def test_rope_theta_in_rope_parameters():
    raw = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    raw["rope_parameters"] = {"rope_type": "default", "rope_theta": 123456.0}
    assert Qwen3Config.from_dict(raw).rope_theta == 123456.0


def test_windows_per_layer():
    assert Qwen3Config.from_dict(TINY_C).layer_windows() == (0, 40, 0, 40)
    raw = dict(TINY_C, layer_types=None)
    assert Qwen3Config.from_dict(raw).layer_windows() == (0, 0, 40, 40)     # from max_window_layers upward
    assert Qwen3Config.from_dict(dict(raw, use_sliding_window=False)).layer_windows() == (0, 0, 0, 0)
    # the switch decides: layer_types may name sliding layers, with the switch off nothing has a window
    assert Qwen3Config.from_dict(dict(TINY_C, use_sliding_window=False)).layer_windows() == (0, 0, 0, 0)
    spec = Qwen3Config.from_dict(TINY_C).to_spec()
    assert [layer.mixer.params["window"] for layer in spec.layers] == [0, 40, 0, 40]


@pytest.mark.parametrize(
    "change,needle",
    [
        ({"num_key_value_heads": 3}, "divisible"),
        ({"head_dim": 24}, "multiple of 16"),
        ({"head_dim": 512}, "at most 256"),
        ({"hidden_act": "gelu"}, "silu"),
        ({"attention_bias": True}, "attention_bias"),
        ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope type"),
        ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
        ({"vocab_size": None}, "vocab_size"),
        ({"layer_types": ["full_attention"]}, "layer_types"),
        ({"use_sliding_window": True, "sliding_window": None, "max_window_layers": 0}, "sliding_window"),
    ],
)
def test_bad_configurations_are_refused(change, needle):
    with pytest.raises(ValueError, match=needle):
        Qwen3Config.from_dict(dict(TINY_A, **change))


def test_overrides_replace_keys():
    assert Qwen3Config.from_dict(TINY_B, {"num_hidden_layers": 1}).num_hidden_layers == 1


def test_registry(tmp_path):
    assert "Qwen3ForCausalLM" in supported_architectures()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}) is Qwen3Config
    assert resolve_architecture({"model_type": "QWEN3"}) is Qwen3Config
    with pytest.raises(ValueError, match="unsupported architecture.*supported: .*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})
    with pytest.raises(ValueError, match="neither"):
        resolve_architecture({})
    with pytest.raises(FileNotFoundError):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ValueError, match="not valid JSON"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(tmp_path).hidden_size == 96


def test_round_trip_through_config_json():
    for raw in CONFIGS.values():
        config = Qwen3Config.from_dict(raw)
        assert Qwen3Config.from_dict(config.to_dict()) == config


def test_schedule_validation():
    from rapid_llm_b200.config import ScheduleEntry
    import dataclasses

    spec = Qwen3Config.from_dict(TINY_A).to_spec()
    twice = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)))
    twice.validate()
    with pytest.raises(ValueError, match="does not run before"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0, cache_from=1), ScheduleEntry(1))).validate()
    with pytest.raises(ValueError, match="names layer"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(5),)).validate()


def test_the_entry_point_refuses_options_of_what_is_not_built():
    """The reference's constructor options are accepted at their neutral values; anything that asks
    for quantisation or more than one GPU is refused before any work, never ignored."""
    from rapid_llm_b200 import LLM

    for option in (dict(quantization="fp8"), dict(tensor_parallel_size=2), dict(data_parallel_size=2),
                   dict(enable_expert_parallel=True), dict(kv_cache_dtype="fp8")):
        with pytest.raises(ValueError) as caught:
            LLM("/nonexistent", **option)
        assert next(iter(option)) in str(caught.value)
