"""From a model folder (or a configuration and a seed) to a loaded model on the device."""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from mini_engine_b200.config.registry import Architecture, architecture_for, load_model_config
from mini_engine_b200.parts.model import DecoderModel
from mini_engine_b200.weights.loader import load_weights, place_tensors
from mini_engine_b200.weights.random_init import random_tensors


def load_model(folder: str | Path, dtype: torch.dtype, device: str = "cuda") -> tuple[Architecture, Any, DecoderModel]:
    """Read ``config.json``, choose the model by its ``architectures`` entry, load the
    safetensors by tensor name (src/mini_engine/engine.py:112-134 of YuvGev00/mini-engine,
    without a hub download: the folder must be local)."""
    arch, config = load_model_config(folder)
    model = DecoderModel(arch.build_spec(config))
    model.load(load_weights(folder, model.weight_specs(), dtype, device))
    return arch, config, model


def random_model(
    config: Any,
    seed: int,
    dtype: torch.dtype,
    device: str = "cuda",
    scale: float = 1.0,
    store: torch.dtype | None = None,
) -> DecoderModel:
    """A model with seeded random weights made directly on the device (no folder).  ``store`` is
    the dtype the values are rounded to when they are made (default: the compute dtype); a float32
    model made with ``store=torch.bfloat16`` holds exactly the bfloat16 model's weights."""
    arch = architecture_for(config.architecture)
    model = DecoderModel(arch.build_spec(config))
    specs = model.weight_specs()
    if store is None:
        store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    tensors = {}
    for spec in specs:  # one tensor at a time keeps the peak at one float32 copy of the largest
        if spec.alias_of is None:
            tensors.update(random_tensors([spec], seed, store, device, scale))
    model.load(place_tensors(tensors, specs, dtype, device))
    return model
