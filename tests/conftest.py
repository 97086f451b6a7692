"""Shared fixtures: tiny model folders with seeded random weights, made in temporary folders."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# Largest relative error that the replay comparisons of a run reached, by dtype; printed at the
# end of the run so that the tolerances can be kept close to what the kernels really do.
WORST_ERRORS: dict[str, float] = {}


def note_error(kind: str, value: float) -> None:
    WORST_ERRORS[kind] = max(WORST_ERRORS.get(kind, 0.0), value)


def pytest_terminal_summary(terminalreporter):
    if WORST_ERRORS:
        terminalreporter.write_line(
            "worst relative logit errors: " + ", ".join(f"{k}={v:.3g}" for k, v in sorted(WORST_ERRORS.items()))
        )


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def make_model_folder(tmp_path_factory, name: str, seed: int, dtype=torch.float32, scale: float = 1.0, raw=None):
    from tiny_configs import CONFIGS

    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.weights import write_random_model

    folder = tmp_path_factory.mktemp(f"tiny_{name}_{seed}")
    cfg = Qwen3Config.from_dict(raw or CONFIGS[name])
    write_random_model(folder, cfg, seed, dtype, scale=scale)
    return folder


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Tiny A and B with the nominal init (N(0, 0.02) matrices), float32 storage."""
    return {name: make_model_folder(tmp_path_factory, name, seed=11) for name in ("A", "B", "C", "D")}


@pytest.fixture(scope="session")
def peaked_model_folders(tmp_path_factory):
    """The same sizes with ten times wider matrices: logits are peaked, so an argmax cannot
    flip on rounding alone (the reference widens its test model's init for the same reason,
    tests/conftest.py:25-27 of YuvGev00/mini-engine)."""
    return {name: make_model_folder(tmp_path_factory, name, seed=12, scale=10.0) for name in ("A", "B", "C", "D")}


def load_plain(folder):
    """Weights and config of a folder for the plain implementation, read with the
    safetensors package (not with the product's own reader)."""
    import plain_qwen3
    from safetensors.torch import load_file

    return load_file(str(Path(folder) / "model.safetensors")), plain_qwen3.read_config(folder)
