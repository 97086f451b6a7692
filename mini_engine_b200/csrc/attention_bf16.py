"""Host side of the bfloat16 tensor-core attention kernels (placeholder until bound)."""

from __future__ import annotations


def supports(head_dim: int, heads: int, kv_heads: int) -> bool:
    return False
