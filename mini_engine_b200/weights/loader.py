"""Loading a model's tensors by checkpoint name.

Every part of a model declares the tensors it needs as :class:`WeightSpec` (full name,
shape and role).  ``load_weights`` checks the whole folder against the whole list first
and raises **one** :class:`WeightError` that lists every missing tensor, every unexpected
tensor and every wrong shape; only then does it move bytes.

Roles decide what a tensor is kept as on the device:

* ``matrix`` (projections, embeddings, heads): the engine's compute dtype, bfloat16 or
  float32;
* ``vector`` (norm weights and other small per-channel tensors): float32 always.  A
  tensor stored in 32-bit therefore stays 32-bit, and a bfloat16 one widens exactly;
* ``table`` (integer lookup tables): int32.

The reference loads with ``load_state_dict(strict=True)`` and then casts the whole module
(src/mini_engine/model.py:190-195, src/mini_engine/engine.py:63 of YuvGev00/mini-engine).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Iterable

import torch

from mini_engine_b200.weights.safetensors_io import read_folder_index

# Buffers that some exporters write although they are derived values, never parameters.
_IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightError(RuntimeError):
    """The checkpoint does not fit the model; the message lists every mismatch."""

    def __init__(self, missing: list[str], unexpected: list[str], wrong_shape: list[str], other: list[str]):
        self.missing, self.unexpected, self.wrong_shape, self.other = missing, unexpected, wrong_shape, other
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if other:
            lines.append("  " + "; ".join(other))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class WeightSpec:
    name: str  # full checkpoint name
    shape: tuple[int, ...]
    role: str = "matrix"  # "matrix", "vector" or "table"
    init: str = "normal"  # random-weights mode: "normal" (N(0, 0.02)) or "ones_normal" (1 + N(0, 0.1))
    alias_of: str | None = None  # tied tensor: use that tensor's storage; a stored copy is ignored


def _target_dtype(role: str, compute: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return compute
    if role == "vector":
        return torch.float32
    if role == "table":
        return torch.int32
    raise ValueError(f"unknown weight role {role!r}")


def check_specs(specs: Iterable[WeightSpec], entries: dict[str, tuple[torch.dtype, tuple[int, ...]]]) -> None:
    """Raise one WeightError for everything that does not fit; return silently otherwise."""
    specs = list(specs)
    wanted = {s.name: s for s in specs}
    missing, wrong, other = [], [], []
    for spec in specs:
        if spec.alias_of is not None:
            if spec.alias_of not in wanted:
                other.append(f"{spec.name} is tied to {spec.alias_of}, which the model does not declare")
            continue
        if spec.name not in entries:
            missing.append(spec.name)
            continue
        dtype, shape = entries[spec.name]
        if tuple(shape) != tuple(spec.shape):
            wrong.append(f"{spec.name}: file has {list(shape)}, model wants {list(spec.shape)}")
        integer = not (dtype.is_floating_point)
        if integer != (spec.role == "table"):
            other.append(f"{spec.name}: stored as {dtype}, which does not fit its role '{spec.role}'")
    unexpected = sorted(
        name for name in entries if name not in wanted and not name.endswith(_IGNORED_SUFFIXES)
    )
    if missing or unexpected or wrong or other:
        raise WeightError(sorted(missing), unexpected, wrong, other)


def load_weights(
    folder: str | Path, specs: Iterable[WeightSpec], compute: torch.dtype, device: torch.device | str
) -> dict[str, torch.Tensor]:
    """Name -> device tensor for every spec; tied names share one storage."""
    specs = list(specs)
    where = read_folder_index(folder)
    entries = {name: opened.entries[name] for name, opened in where.items()}
    check_specs(specs, entries)
    out: dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.alias_of is None:
            host = where[spec.name].tensor(spec.name)
            out[spec.name] = host.to(device=device, dtype=_target_dtype(spec.role, compute)).contiguous()
    for spec in specs:
        if spec.alias_of is not None:
            out[spec.name] = out[spec.alias_of]
    return out


def place_tensors(
    tensors: dict[str, torch.Tensor], specs: Iterable[WeightSpec], compute: torch.dtype, device
) -> dict[str, torch.Tensor]:
    """The same checks and casts for tensors that are already in memory (random weights)."""
    specs = list(specs)
    check_specs(specs, {n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()})
    out = {
        s.name: tensors[s.name].to(device=device, dtype=_target_dtype(s.role, compute)).contiguous()
        for s in specs
        if s.alias_of is None
    }
    for s in specs:
        if s.alias_of is not None:
            out[s.name] = out[s.alias_of]
    return out
