"""Sampling: per-request options and the device sampler."""

from mini_engine_b200.sampling.params import SamplingParams

__all__ = ["SamplingParams"]
