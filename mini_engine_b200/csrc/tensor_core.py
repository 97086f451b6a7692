"""Host side of the TMA + tcgen05 matrix product (placeholder until the kernel is bound)."""

from __future__ import annotations


def supports(outs: int, inner: int) -> bool:
    return False


def choose_splits(tokens: int, outs: int, inner: int, max_splits: int = 8) -> int:
    return 1
