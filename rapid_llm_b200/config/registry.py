"""One registry from an architecture's name to what builds its model.

The reference keys its registry on ``config.json``'s ``model_type`` and imports
the model class lazily (``rapid_llm/models/registry.py:20-78``); its cheap sniff
of the file has three distinct errors (``rapid_llm/models/config.py:42-62``).
Here the key is the first entry of ``architectures`` with ``model_type`` as the
fallback, and the value is the architecture's configuration class, whose
``to_spec()`` yields the layer list the generic model runs.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Protocol

from .model_spec import ModelSpec


class ArchitectureConfig(Protocol):
    """What an architecture has to provide to be served."""

    architecture: str
    model_type: str

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], overrides: Mapping[str, Any] | None = None): ...

    def to_dict(self) -> dict[str, Any]: ...

    def to_spec(self) -> ModelSpec: ...


_BY_ARCHITECTURE: dict[str, type] = {}
_BY_MODEL_TYPE: dict[str, type] = {}


def register_architecture(config_class: type) -> type:
    """Make an architecture loadable; usable as a class decorator."""
    _BY_ARCHITECTURE[config_class.architecture] = config_class
    _BY_MODEL_TYPE[str(config_class.model_type).lower()] = config_class
    return config_class


def supported_architectures() -> list[str]:
    return sorted(_BY_ARCHITECTURE)


def resolve_architecture(raw: Mapping[str, Any]) -> type:
    """The configuration class for a parsed ``config.json``."""
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for name in names:
        if name in _BY_ARCHITECTURE:
            return _BY_ARCHITECTURE[name]
    model_type = raw.get("model_type")
    if model_type is not None and str(model_type).lower() in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[str(model_type).lower()]
    if not names and model_type is None:
        raise ValueError("config.json names neither 'architectures' nor 'model_type'")
    raise ValueError(
        f"unsupported architecture {list(names) or model_type!r}; "
        f"supported: {', '.join(supported_architectures())}"
    )


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {Path(model_dir)}")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ValueError(f"{path} is not valid JSON: {exc}") from exc
    if not isinstance(raw, dict):
        raise ValueError(f"{path} does not hold a JSON object")
    return raw


def load_config(model_dir: str | Path, overrides: Mapping[str, Any] | None = None):
    """Read ``config.json`` of a model folder into its architecture's configuration."""
    raw = read_config_json(model_dir)
    return resolve_architecture(raw).from_dict(raw, overrides)
