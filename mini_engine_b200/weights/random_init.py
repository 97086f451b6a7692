"""Seeded random weights, generated tensor by tensor *by name*.

Each value is a pure function of (seed, tensor name, element index): a 64-bit counter hash
(the splitmix64 finaliser) evaluated with wrapping integer arithmetic, which gives the same
bits on the host and on the device and does not depend on the order in which tensors are
made.  A folder written here on any machine, the engine's in-memory random model
(``LLMEngine.from_random``, made on the device) and any other reader of the folder therefore
hold the same numbers.  A standard normal value is the centred sum of twelve 16-bit uniform
fields of three hashes (Irwin-Hall: mean 0, variance 1, support +-6; no logarithm or cosine,
whose last bits differ between host and device libraries).  Initialisation: matrices and
embeddings N(0, 0.02); norm weights 1 + N(0, 0.1).  The reference has no such mode; its tests
build a random model through a library (tests/conftest.py:13-35 of YuvGev00/mini-engine).
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
_CHUNK = 1 << 24  # elements hashed at a time: bounds the int64 temporaries of a large matrix


def _signed(value: int) -> int:
    value &= 0xFFFF_FFFF_FFFF_FFFF
    return value - (1 << 64) if value >= (1 << 63) else value


_GOLDEN = _signed(0x9E37_79B9_7F4A_7C15)
_MIX_1 = _signed(0xBF58_476D_1CE4_E5B9)
_MIX_2 = _signed(0x94D0_49BB_1331_11EB)


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return _signed(int.from_bytes(digest, "little"))


def _shift_right(x: torch.Tensor, bits: int) -> torch.Tensor:
    """Logical right shift of int64 values (``>>`` alone copies the sign bit down)."""
    return (x >> bits) & ((1 << (64 - bits)) - 1)


def _hash64(counters: torch.Tensor, key: int) -> torch.Tensor:
    x = counters * _GOLDEN + key  # int64 arithmetic wraps, on the host and on the device alike
    x = (x ^ _shift_right(x, 30)) * _MIX_1
    x = (x ^ _shift_right(x, 27)) * _MIX_2
    return x ^ _shift_right(x, 31)


def standard_normal(count: int, key: int, device="cpu", first: int = 0) -> torch.Tensor:
    """``count`` float32 values for element indices ``first ..``; see the module docstring."""
    out = torch.empty(count, dtype=torch.float32, device=device)
    for begin in range(0, count, _CHUNK):
        n = min(_CHUNK, count - begin)
        index = torch.arange(first + begin, first + begin + n, dtype=torch.int64, device=device) * 3
        total = torch.zeros(n, dtype=torch.int64, device=device)
        for j in range(3):
            bits = _hash64(index + j, key)
            for field in range(4):
                total += _shift_right(bits, 16 * field) & 0xFFFF
        # twelve uniform fields on 0..65535: mean 6 * 65535, variance 12 * (65536^2 - 1) / 12
        out[begin : begin + n] = (total - 6 * 65535).to(torch.float32) * (1.0 / 65536.0)
    return out


def random_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype, device="cpu", scale: float = 1.0):
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    count = 1
    for extent in spec.shape:
        count *= extent
    values = standard_normal(count, _seed_for(seed, spec.name), device).view(spec.shape)
    if spec.init == "ones_normal":
        values = values * NORM_STD  # two roundings, the same two everywhere (no fused multiply-add)
        values = values + 1.0
    else:
        values = values * (MATRIX_STD * scale)
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
