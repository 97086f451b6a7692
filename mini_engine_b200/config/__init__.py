"""Typed configuration: the model's own ``config.json`` keys and the engine's options."""

from mini_engine_b200.config.engine_config import EngineConfig
from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from mini_engine_b200.config.qwen3 import Qwen3Config
from mini_engine_b200.config.registry import (
    Architecture,
    architecture_for,
    load_model_config,
    register_architecture,
    registered_architectures,
)

__all__ = [
    "Architecture",
    "EngineConfig",
    "LayerSpec",
    "ModelSpec",
    "OrderEntry",
    "PartSpec",
    "Qwen3Config",
    "architecture_for",
    "load_model_config",
    "register_architecture",
    "registered_architectures",
]
