"""Options of the engine, with the names and meanings of the reference's ``EngineConfig``
(src/mini_engine/engine.py:22-36 of YuvGev00/mini-engine).

Dropped on purpose: ``speculative`` and ``attention_backend`` (there is one attention path
and no speculative decoding here) and ``device`` (the engine runs on ``cuda:0`` only).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class EngineConfig:
    block_size: int = 16  # tokens per KV page
    num_blocks: int = 256  # pages in the pool of every cache group
    max_num_seqs: int = 16  # requests that may run at the same time
    max_num_batched_tokens: int = 2048  # token budget of one step
    max_model_len: int = 4096  # prompt + generated tokens of one request
    enable_prefix_caching: bool = True
    dtype: torch.dtype = torch.float32  # torch.float32 or torch.bfloat16
    seed: int = 0  # seed of temperature sampling
    cuda_graphs: bool = True  # replay captured graphs for decode-only steps
    # When set (0 < f <= 1), num_blocks is ignored and the pool takes this fraction of the device
    # memory that is free after the weights are loaded.  The reference sizes by num_blocks only.
    kv_memory_fraction: float | None = None
    # Launch the decode step after the current one before the current one's token ids are read
    # (needs cuda_graphs).  The tokens are the same either way; off is for comparing.  Not in the
    # reference, whose steps are strictly one after the other.
    overlap_steps: bool = True

    def __post_init__(self) -> None:
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be torch.float32 or torch.bfloat16, got {self.dtype}")
        for name in ("block_size", "num_blocks", "max_num_seqs", "max_num_batched_tokens", "max_model_len"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be positive")
        if self.kv_memory_fraction is not None and not 0.0 < self.kv_memory_fraction <= 1.0:
            raise ValueError("kv_memory_fraction must lie in (0, 1]")
