"""Sampling options of one request, with the reference's names and meanings
(src/mini_engine/sequence.py:10-20 of YuvGev00/mini-engine)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 64  # stop after this many generated tokens
    temperature: float = 0.0  # 0.0 means greedy
    ignore_eos: bool = False  # keep generating through an end-of-sequence token

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
