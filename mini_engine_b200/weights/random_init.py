"""Seeded random weights, generated tensor by tensor *by name*.

Each tensor's values depend only on (seed, tensor name, shape), never on the order in which
tensors are made, so a folder written here, the engine's in-memory random model and any
other reader of the folder hold the same numbers.  Initialisation: matrices and embeddings
N(0, 0.02); norm weights 1 + N(0, 0.1).  The reference has no such mode; its tests build a
random model through a library (tests/conftest.py:13-35 of YuvGev00/mini-engine).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Iterable

import torch

from mini_engine_b200.weights.loader import WeightSpec
from mini_engine_b200.weights.safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return int.from_bytes(digest, "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype, device="cpu", scale: float = 1.0):
    generator = torch.Generator(device=device).manual_seed(_seed_for(seed, spec.name))
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    values = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device)
    if spec.init == "ones_normal":
        values = 1.0 + NORM_STD * values
    else:
        values = MATRIX_STD * scale * values
    return values.to(dtype)


def random_tensors(
    specs: Iterable[WeightSpec], seed: int, dtype: torch.dtype, device="cpu", scale: float = 1.0
) -> dict[str, torch.Tensor]:
    """``scale`` widens the matrices' standard deviation (tests use it to make logits
    peaked, so that an argmax cannot flip on rounding alone)."""
    return {
        s.name: random_tensor(s, seed, dtype, device, scale) for s in specs if s.alias_of is None
    }


def write_random_model(
    folder: str | Path,
    config: Any,
    seed: int,
    dtype: torch.dtype = torch.bfloat16,
    scale: float = 1.0,
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a typed configuration.

    The architecture is looked up by ``config.architecture``; its parts say which tensors
    exist.  Returns the folder.
    """
    from mini_engine_b200.config.registry import architecture_for
    from mini_engine_b200.parts.model import declared_weights

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = architecture_for(config.architecture)
    specs = declared_weights(arch.build_spec(config))
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", random_tensors(specs, seed, dtype, scale=scale))
    return folder
