"""Configuration: model specification, architecture registry, engine sizes."""

from .engine_config import EngineConfig, parse_dtype
from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen3 import Qwen3Config
from .registry import (
    load_config,
    read_config_json,
    register_architecture,
    resolve_architecture,
    supported_architectures,
)

register_architecture(Qwen3Config)

__all__ = [
    "EngineConfig",
    "LayerSpec",
    "ModelSpec",
    "PartSpec",
    "Qwen3Config",
    "ScheduleEntry",
    "load_config",
    "parse_dtype",
    "read_config_json",
    "register_architecture",
    "resolve_architecture",
    "supported_architectures",
]
