"""The plain implementation against the reference's own model code (stored outputs) and
against itself in float64."""

from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import load_plain, make_model_folder
from tiny_configs import CONFIGS, random_ids

GOLDEN = Path(__file__).parent / "golden"
GOLDEN_SEED = 7
GOLDEN_LEN = {"A": 33, "B": 41, "C": 50, "D": 37}


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_plain_matches_reference_model_code(name, tmp_path_factory):
    """tests/golden/make_golden.py ran YuvGev00/mini-engine's model on CPU in float32."""
    folder = make_model_folder(tmp_path_factory, name, seed=GOLDEN_SEED)
    weights, cfg = load_plain(folder)
    prompt = random_ids(GOLDEN_SEED, GOLDEN_LEN[name], cfg["vocab"])
    stored = np.fromfile(GOLDEN / f"tiny_{name}_logits.f32", dtype="<f4").reshape(len(prompt), cfg["vocab"])
    ours = plain.forward_logits(weights, cfg, prompt).numpy()
    np.testing.assert_allclose(ours, stored, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_float32_close_to_float64(name, model_folders):
    weights, cfg = load_plain(model_folders[name])
    prompt = random_ids(3, 50, cfg["vocab"])
    f32 = plain.forward_logits(weights, cfg, prompt, torch.float32)
    f64 = plain.forward_logits(weights, cfg, prompt, torch.float64)
    assert (f32.double() - f64).abs().max() < 2e-5


def test_read_config_defaults(tmp_path):
    from tiny_configs import write_config

    raw = dict(CONFIGS["A"])
    del raw["head_dim"], raw["rope_theta"]
    write_config(tmp_path, raw)
    cfg = plain.read_config(tmp_path)
    assert cfg["head_dim"] == 16 and cfg["theta"] == 10000.0


def test_causal_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    full = plain.causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 0.0, 7.0  # later keys must not influence earlier queries
    assert torch.equal(plain.causal_attention(q, k2, v2)[:4], full[:4])
    assert torch.allclose(full[0], v[0].repeat_interleave(2, dim=0))  # first query sees only key 0
    windowed = plain.causal_attention(q, k, v, window=1)
    assert torch.allclose(windowed, v.repeat_interleave(2, dim=1))  # window 1: only itself


def test_rope_position_zero_is_identity_and_norm_preserved():
    x = torch.randn(3, 2, 16)
    cos, sin = plain.rope_angles(torch.tensor([0, 5, 900]), 16, 10000.0, torch.float32)
    y = plain.apply_rope(x, cos, sin)
    assert torch.allclose(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_sampling_reference():
    logits = torch.tensor([0.0, 3.0, 3.0, -1.0])
    assert plain.sample_from_logits(logits, 0.0, 0.5) == 1
    assert plain.sample_from_logits(logits, 1.0, 0.0) == 0
    assert plain.sample_from_logits(logits, 1.0, 0.999999) == 3
