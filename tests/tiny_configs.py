"""The two tiny Qwen3-dense configurations that the tests run, and seeded inputs.

They differ in every size and option: layers, width, head count and group size, head size,
feed-forward width (no power of two in B), vocabulary, rope theta, the norms' eps, tied or
untied head, and the page size they are run with.
"""

from __future__ import annotations

import json
import random
from pathlib import Path

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "intermediate_size": 160,
    "vocab_size": 384,
    "rope_parameters": {"rope_type": "default", "rope_theta": 1000000.0},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 1024,
    "hidden_act": "silu",
}
# A third size whose head_dim (64) the bfloat16 tensor-core attention kernels take, so that the
# whole-model replays exercise them too (A and B, at 16 and 32, use the generic kernel).
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 136,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "intermediate_size": 200,
    "vocab_size": 320,
    "rope_theta": 500000.0,
    "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 2048,
    "hidden_act": "silu",
}
# A fourth size with head_dim 128, the size at which the tcgen05 attention kernel and the
# vector paths of the q/k norm + rotation kernel run, one KV head for four query heads, and
# pages of 32 tokens.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 192,
    "num_attention_heads": 4,
    "num_key_value_heads": 1,
    "head_dim": 128,
    "intermediate_size": 384,
    "vocab_size": 300,
    "rope_theta": 20000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 2048,
    "hidden_act": "silu",
}
# One layer of Qwen3-8B's sizes (hidden 4096, 32 / 8 heads of 128, intermediate 12288) under a
# small vocabulary: the products, norms and attention run at the sizes the benchmark runs them,
# the CTA-pair kernels and their split and stacked relatives included, against the plain
# implementation.  Not in CONFIGS: only the tests that ask for it by name pay for it.
LAYER_OF_8B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 1,
    "hidden_size": 4096,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "intermediate_size": 12288,
    "vocab_size": 1000,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 4096,
    "hidden_act": "silu",
}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 32, "8B": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def random_ids(seed: int, count: int, vocab: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


def write_config(folder: Path, raw: dict) -> None:
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=2))
