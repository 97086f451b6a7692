"""A small, whole inference engine for one NVIDIA B200: from a model folder to tokens.

Public names follow YuvGev00/mini-engine (src/mini_engine/__init__.py:3-6).
"""

from mini_engine_b200.config.engine_config import EngineConfig
from mini_engine_b200.engine.sequence import Sequence
from mini_engine_b200.sampling.params import SamplingParams

__all__ = ["EngineConfig", "EngineStats", "LLMEngine", "SamplingParams", "Sequence"]


def __getattr__(name: str):
    if name in ("LLMEngine", "EngineStats"):
        from mini_engine_b200.engine import llm_engine

        return getattr(llm_engine, name)
    raise AttributeError(name)
