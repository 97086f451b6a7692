"""One registry from an architecture's name (``config.json: architectures[0]``) to its
typed configuration and to the function that lays the model out as a :class:`ModelSpec`.

The reference has no registry: it checks ``model_type`` and builds its only model
(src/mini_engine/model.py:37-38 of YuvGev00/mini-engine).  Here another architecture is
added by one ``register_architecture`` call from its own module; nothing else changes.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from mini_engine_b200.config.model_spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[Path], Any]  # model folder -> typed configuration
    build_spec: Callable[[Any], ModelSpec]  # typed configuration -> parts, layer by layer
    config_type: type | None = None


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def architecture_for(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise KeyError(
            f"no architecture {name!r} is registered; registered: {', '.join(sorted(_ARCHITECTURES))}"
        )
    return _ARCHITECTURES[name]


def architecture_of_folder(folder: str | Path) -> Architecture:
    config_file = Path(folder) / "config.json"
    if not config_file.is_file():
        raise FileNotFoundError(f"{folder} has no config.json")
    raw = json.loads(config_file.read_text())
    names = raw.get("architectures") or []
    if not names:
        raise KeyError(f"{config_file} has no 'architectures' entry to choose a model by")
    return architecture_for(names[0])


def load_model_config(folder: str | Path) -> tuple[Architecture, Any]:
    """The architecture that ``config.json`` names and its typed configuration."""
    arch = architecture_of_folder(folder)
    return arch, arch.read_config(Path(folder))


def _ensure_builtin() -> None:
    # The built-in architecture registers itself on import; importing here (not at the top)
    # keeps this module free of a cycle with the model modules.
    import mini_engine_b200.models  # noqa: F401
