"""Typed configuration of the Qwen3 dense decoder, read from its own ``config.json`` keys.

Follows ``ModelConfig.from_hf`` of YuvGev00/mini-engine (src/mini_engine/model.py:21-56):
the same eleven fields, the same defaults (``head_dim`` = ``hidden_size //
num_attention_heads``, ``rope_theta`` from ``rope_parameters`` else the top level else
10000.0) and the same three rejections (another ``model_type``, a RoPE type other than
``default``, sliding-window attention).  Keys that the reference ignores silently but that
would change the arithmetic (``attention_bias``, ``hidden_act``, a legacy ``rope_scaling``)
are rejected here, because a silently wrong model is worse than an error.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that this engine cannot run, with the key that is at fault."""


def _require(raw: Mapping[str, Any], key: str, kind: type | tuple[type, ...]) -> Any:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks the key {key!r}")
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config.json key {key!r} must be {kind}, got {value!r}")
    return value


def _as_id_tuple(value: Any) -> tuple[int, ...]:
    """``eos_token_id`` may be absent, one id or a list (src/mini_engine/engine.py:302-307)."""
    if value is None:
        return ()
    if isinstance(value, int):
        return (value,)
    return tuple(int(v) for v in value)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Qwen3ForCausalLM"

    def __post_init__(self) -> None:
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
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for rotate-half RoPE, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], eos_override: Any = None) -> "Qwen3Config":
        model_type = raw.get("model_type", "qwen3")
        if model_type != "qwen3":
            raise ConfigError(f"only model_type 'qwen3' is supported, got {model_type!r}")
        rope = raw.get("rope_parameters") or {}
        if rope.get("rope_type", "default") != "default":
            raise ConfigError(f"only the default RoPE is supported, got {rope.get('rope_type')!r}")
        legacy = raw.get("rope_scaling")
        if legacy and legacy.get("rope_type", legacy.get("type", "default")) != "default":
            raise ConfigError(f"rope_scaling {legacy!r} is not supported")
        if raw.get("use_sliding_window", False):
            raise ConfigError("sliding-window attention is not supported for Qwen3 dense")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: the projections have no bias")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act must be 'silu', got {raw.get('hidden_act')!r}")
        heads = _require(raw, "num_attention_heads", int)
        hidden = _require(raw, "hidden_size", int)
        head_dim = raw.get("head_dim") or hidden // heads
        eos = eos_override if eos_override is not None else raw.get("eos_token_id")
        return cls(
            vocab_size=_require(raw, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size", int),
            num_hidden_layers=_require(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=_require(raw, "num_key_value_heads", int),
            head_dim=int(head_dim),
            rms_norm_eps=float(_require(raw, "rms_norm_eps", (int, float))),
            rope_theta=float(rope.get("rope_theta", raw.get("rope_theta", 10000.0))),
            max_position_embeddings=_require(raw, "max_position_embeddings", int),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            eos_token_ids=_as_id_tuple(eos),
        )

    @classmethod
    def from_folder(cls, folder: str | Path) -> "Qwen3Config":
        """``config.json`` of a model folder; end-of-sequence ids come from
        ``generation_config.json`` when that file exists, else from ``config.json``
        (src/mini_engine/engine.py:130-133)."""
        folder = Path(folder)
        raw = json.loads((folder / "config.json").read_text())
        eos = None
        generation = folder / "generation_config.json"
        if generation.is_file():
            eos = json.loads(generation.read_text()).get("eos_token_id")
        return cls.from_dict(raw, eos_override=eos)

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back to this configuration."""
        out = asdict(self)
        eos = out.pop("eos_token_ids")
        out["eos_token_id"] = list(eos) if len(eos) != 1 else eos[0]
        if not eos:
            out["eos_token_id"] = None
        out["architectures"] = [self.architecture]
        out["model_type"] = "qwen3"
        out["hidden_act"] = "silu"
        out["attention_bias"] = False
        out["use_sliding_window"] = False
        return out
