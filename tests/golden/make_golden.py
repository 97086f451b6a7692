"""Makes tests/golden/*.f32: logits of YuvGev00/mini-engine's own model code on CPU.

The reference's ``Qwen3ForCausalLM`` is built directly from numbers (no library model code),
loaded with this repository's seeded by-name random weights through its own
``load_hf_state_dict``, and run in float32 on CPU through its own engine pieces exactly as
its tests/test_parity.py:67-77 does: schedule one request, ``_prepare``, call the model with
``logits_index = arange``.  The outputs (a few tens of KB) are committed; the test
``tests/test_plain.py`` checks the plain implementation against them.

    MINI_ENGINE_REF=/path/to/mini-engine/src python tests/golden/make_golden.py
"""

from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))
if "MINI_ENGINE_REF" not in os.environ:
    sys.exit("set MINI_ENGINE_REF to the src folder of a YuvGev00/mini-engine checkout")
sys.path.insert(0, os.environ["MINI_ENGINE_REF"])

from tiny_configs import CONFIGS, PAGE_SIZE, random_ids  # noqa: E402

from mini_engine_b200.config import Qwen3Config  # noqa: E402
from mini_engine_b200.weights import write_random_model  # noqa: E402

GOLDEN_SEED = 7
GOLDEN_LEN = {"A": 33, "B": 41, "C": 50, "D": 37}


def main() -> None:
    from mini_engine.engine import EngineConfig, LLMEngine
    from mini_engine.model import ModelConfig, Qwen3ForCausalLM
    from safetensors.torch import load_file

    for name, raw in CONFIGS.items():
        cfg = Qwen3Config.from_dict(raw)
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(folder, cfg, GOLDEN_SEED, torch.float32)
            state = load_file(os.path.join(folder, "model.safetensors"))
        ref_cfg = ModelConfig(
            vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
            num_layers=cfg.num_hidden_layers, num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_norm_eps,
            rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position_embeddings,
            tie_word_embeddings=cfg.tie_word_embeddings,
        )  # fmt: skip
        model = Qwen3ForCausalLM(ref_cfg)
        model.load_hf_state_dict(state)
        engine = LLMEngine(model, EngineConfig(block_size=PAGE_SIZE[name], num_blocks=64, max_model_len=256))
        prompt = random_ids(GOLDEN_SEED, GOLDEN_LEN[name], cfg.vocab_size)
        engine.add_request(prompt)
        batch = engine.scheduler.schedule()
        ids, pos, meta, _ = engine._prepare(batch)
        with torch.inference_mode():
            logits = engine.model(ids, pos, engine.kv_caches, meta, torch.arange(len(prompt)))
        out = HERE / f"tiny_{name}_logits.f32"
        logits.numpy().astype("<f4").tofile(out)
        print(name, tuple(logits.shape), float(logits.abs().max()), "->", out.name)


if __name__ == "__main__":
    main()
