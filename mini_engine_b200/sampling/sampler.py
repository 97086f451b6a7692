"""Greedy and temperature sampling on the device.

The reference computes ``argmax`` for temperature 0 and otherwise draws from
``softmax(logits / max(T, 1e-5))`` with one generator for the whole engine, so that a
request's sampled tokens depend on what else is in the batch
(src/mini_engine/engine.py:80,282-291 of YuvGev00/mini-engine).  Here every draw uses a
uniform number that is a pure function of (engine seed, request id, index of the generated
token), so a request's stream is the same alone, batched, preempted or resumed.
"""

from __future__ import annotations

import hashlib
import struct
from typing import Sequence as Seq

import torch

from mini_engine_b200.csrc import ops


def uniform_for(seed: int, request_id: int, token_index: int) -> float:
    """A number in [0, 1) with 24 random bits, the same on every run and machine."""
    digest = hashlib.blake2b(struct.pack("<qqq", seed, request_id, token_index), digest_size=8).digest()
    return (int.from_bytes(digest, "little") >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, seed: int, max_rows: int, device: str | torch.device = "cuda"):
        self.seed = seed
        self.device = torch.device(device)
        self._host = torch.empty((2, max_rows), dtype=torch.float32).pin_memory()
        self._params = torch.empty((2, max_rows), dtype=torch.float32, device=self.device)
        self._tokens = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._tokens_host = torch.empty(max_rows, dtype=torch.int32).pin_memory()

    def sample(
        self,
        logits: torch.Tensor,
        temperatures: Seq[float],
        request_ids: Seq[int],
        token_indices: Seq[int],
    ) -> list[int]:
        """One token per row of ``logits [rows, vocab]`` (float32, on the device)."""
        rows = logits.shape[0]
        if rows == 0:
            return []
        out = self._tokens[:rows]
        if all(t == 0 for t in temperatures):
            ops.sample(logits, None, None, out)
        else:
            host = self._host
            for i in range(rows):
                host[0, i] = temperatures[i]
                host[1, i] = uniform_for(self.seed, request_ids[i], token_indices[i]) if temperatures[i] else 0.0
            self._params[:, :rows].copy_(host[:, :rows], non_blocking=True)
            temps = self._params[0, :rows]
            uniforms = self._params[1, :rows]
            ops.sample(logits, temps, uniforms, out)
        self._tokens_host[:rows].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._tokens_host[:rows].tolist()
