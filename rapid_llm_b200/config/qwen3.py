"""Typed configuration of the Qwen3 dense decoder, read from ``config.json``.

The reference wraps a ``transformers`` config object and falls through to its
attributes (``rapid_llm/models/config.py:65-417``); its Qwen3 model is two class
flags on the shared skeleton, ``qkv_bias=False`` and ``use_qk_norm=True``
(``rapid_llm/models/qwen3.py:16-18``).  Here the keys are read from the JSON
directly into a dataclass, the keys the reference silently ignores are checked,
and :meth:`Qwen3Config.to_spec` writes the layer list the engine runs.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Mapping

from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config:
    """The keys of a Qwen3 ``config.json`` that shape the computation.

    Defaults follow the reference where it has one: ``num_key_value_heads``
    falls back to the head count (``rapid_llm/models/config.py:171-173``),
    ``head_dim`` to ``hidden_size // num_attention_heads`` with an explicit value
    winning (``:176-178``), ``tie_word_embeddings`` to ``False`` (``:265-267``),
    ``rope_theta`` to 10000 (``:318-335``).  Sizes have no default: a folder
    that omits one is rejected.
    """

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    sliding_window: int | None = None
    use_sliding_window: bool = False
    max_window_layers: int | None = None
    layer_types: tuple[str, ...] = field(default_factory=tuple)
    torch_dtype: str = "bfloat16"

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    _REQUIRED = (
        "vocab_size",
        "hidden_size",
        "intermediate_size",
        "num_hidden_layers",
        "num_attention_heads",
        "max_position_embeddings",
        "rms_norm_eps",
    )

    # ------------------------------------------------------------------ read #
    @classmethod
    def from_dict(
        cls, raw: Mapping[str, Any], overrides: Mapping[str, Any] | None = None
    ) -> "Qwen3Config":
        """Build from the parsed JSON; ``overrides`` replace keys before validation.

        Overrides mirror the reference's ``hf_overrides`` (``rapid_llm/models/config.py:117-131``),
        e.g. ``{"num_hidden_layers": 1}`` runs a trimmed stack through every path.
        Unknown keys are ignored.
        """
        data = dict(raw)
        data.update(overrides or {})
        missing = [key for key in cls._REQUIRED if data.get(key) is None]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")

        heads = int(data["num_attention_heads"])
        hidden = int(data["hidden_size"])
        kv_heads = int(data.get("num_key_value_heads") or heads)
        head_dim = int(data.get("head_dim") or hidden // heads)

        rope = dict(data.get("rope_parameters") or data.get("rope_scaling") or {})
        rope_type = rope.pop("rope_type", rope.pop("type", "default"))
        if rope_type not in ("default", None):
            raise ValueError(
                f"rope type {rope_type!r} is not part of the Qwen3 dense decoder served here "
                "(only 'default')"
            )
        theta = data.get("rope_theta")
        if theta is None:
            theta = rope.get("rope_theta", 10000.0)

        layer_types = tuple(data.get("layer_types") or ())
        dtype = data.get("torch_dtype", data.get("dtype", "bfloat16"))

        config = cls(
            vocab_size=int(data["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(data["intermediate_size"]),
            num_hidden_layers=int(data["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=int(data["max_position_embeddings"]),
            rms_norm_eps=float(data["rms_norm_eps"]),
            rope_theta=float(theta),
            partial_rotary_factor=float(data.get("partial_rotary_factor", 1.0)),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            attention_bias=bool(data.get("attention_bias", False)),
            hidden_act=str(data.get("hidden_act", "silu")),
            sliding_window=(
                None if data.get("sliding_window") is None else int(data["sliding_window"])
            ),
            use_sliding_window=bool(data.get("use_sliding_window", False)),
            max_window_layers=(
                None if data.get("max_window_layers") is None else int(data["max_window_layers"])
            ),
            layer_types=layer_types,
            torch_dtype=str(dtype).replace("torch.", ""),
        )
        config.validate()
        return config

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` a model folder of this configuration carries."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
        }
        for item in fields(self):
            value = getattr(self, item.name)
            if item.name == "layer_types":
                if value:
                    out[item.name] = list(value)
                continue
            if item.name == "max_window_layers" and value is None:
                continue
            out[item.name] = value
        return out

    # -------------------------------------------------------------- validate #
    def validate(self) -> None:
        """Reject what the parts cannot compute, naming the offending numbers.

        The geometry checks are the reference's (``rapid_llm/models/config.py:357-378``);
        the head size must be a multiple of 16 here because the attention
        kernels tile the head dimension in steps of 16.
        """
        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "max_position_embeddings",
        ):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ValueError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                f"num_key_value_heads ({self.num_key_value_heads}) for grouped-query attention"
            )
        if self.head_dim % 16 != 0 or self.head_dim > 256:
            raise ValueError(
                f"head_dim ({self.head_dim}) must be a multiple of 16 and at most 256"
            )
        if self.rms_norm_eps <= 0:
            raise ValueError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_theta <= 0:
            raise ValueError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ValueError(
                f"hidden_act {self.hidden_act!r}: the Qwen3 feed-forward is SwiGLU with silu"
            )
        if self.attention_bias:
            raise ValueError("attention_bias=true is not part of the Qwen3 dense decoder served here")
        rotary = self.rotary_dim
        if rotary <= 0 or rotary % 2 or rotary > self.head_dim:
            raise ValueError(
                f"partial_rotary_factor {self.partial_rotary_factor} gives a rotary width of "
                f"{rotary}, which must be even and within head_dim ({self.head_dim})"
            )
        if self.layer_types:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ValueError(
                    f"layer_types has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers"
                )
            unknown = sorted(set(self.layer_types) - {FULL_ATTENTION, SLIDING_ATTENTION})
            if unknown:
                raise ValueError(f"unknown layer_types entries: {unknown}")
        if not self.use_sliding_window:
            wants_window = False
        elif self.layer_types:
            wants_window = SLIDING_ATTENTION in self.layer_types
        else:
            wants_window = (self.max_window_layers or 0) < self.num_hidden_layers
        if wants_window and (self.sliding_window is None or self.sliding_window < 1):
            raise ValueError(
                "sliding-window layers are configured but sliding_window is "
                f"{self.sliding_window!r}"
            )

    # ------------------------------------------------------------- derived #
    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    def layer_windows(self) -> tuple[int, ...]:
        """Window of each layer in positions, the query's own included; 0 = all keys.

        Windows exist only under ``use_sliding_window`` with a ``sliding_window`` size: the switch is
        the architecture's own, and with it off the size has no meaning whatever else is written.
        Where they exist, ``layer_types`` names the layers that have one; without that key they are
        the layers from ``max_window_layers`` upwards, which is how the architecture's own
        configuration defines these keys.  The reference never reads them for this model and always
        attends over everything (``rapid_llm/engine/kv_cache_spec.py:383-387``), which is what every
        published Qwen3 dense configuration (``use_sliding_window: false``) asks for.
        """
        window = self.sliding_window or 0
        if not self.use_sliding_window or not window:
            return (0,) * self.num_hidden_layers
        if self.layer_types:
            return tuple(
                window if kind == SLIDING_ATTENTION else 0 for kind in self.layer_types
            )
        first = self.max_window_layers if self.max_window_layers is not None else 0
        return tuple(window if index >= first else 0 for index in range(self.num_hidden_layers))

    # ----------------------------------------------------------------- spec #
    def to_spec(self) -> ModelSpec:
        """The layer list of the Qwen3 dense decoder.

        Per layer, in the reference's order (``rapid_llm/models/base.py:231-266``):
        input RMSNorm, attention with per-head q/k RMSNorm before RoPE
        (``:121-165``), post-attention RMSNorm, SwiGLU feed-forward
        (``rapid_llm/modules/mlp.py:52-68``).
        """
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec(
            "rope",
            {
                "head_dim": self.head_dim,
                "rotary_dim": self.rotary_dim,
                "theta": self.rope_theta,
                "max_positions": self.max_position_embeddings,
            },
        )
        windows = self.layer_windows()
        layers = []
        for index in range(self.num_hidden_layers):
            mixer = PartSpec(
                "gqa_attention",
                {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim,
                    "qk_norm": True,
                    "qk_norm_eps": self.rms_norm_eps,
                    "window": windows[index],
                    "scale": self.head_dim**-0.5,
                    "position": position,
                },
            )
            feed_forward = PartSpec(
                "swiglu",
                {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size},
            )
            layers.append(
                LayerSpec(
                    arrangement="prenorm",
                    mixer=mixer,
                    feed_forward=feed_forward,
                    norm=norm,
                    prefix=f"model.layers.{index}.",
                )
            )
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec(
                "token_embedding",
                {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size},
            ),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(index) for index in range(self.num_hidden_layers)),
            final_norm=norm,
            head=PartSpec(
                "lm_head",
                {
                    "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size,
                    "tied": self.tie_word_embeddings,
                },
            ),
            final_norm_prefix="model.norm.",
            embedding_prefix="model.embed_tokens.",
            head_prefix="lm_head.",
        )
        spec.validate()
        return spec
