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
from dataclasses import dataclass
from typing import Sequence as Seq

import torch

from mini_engine_b200.csrc import ops


def uniform_for(seed: int, request_id: int, token_index: int) -> float:
    """A number in [0, 1) with 24 random bits (every value a float32 holds exactly), the same on
    every run and machine.  With 24 bits the smallest step of the cumulative distribution that a
    draw can resolve is 2^-24 (6e-8): a token whose probability is far below that is drawn less
    often than its probability says, or never; over a vocabulary of 150,000 tokens that is the
    tail below one part in ten million, which sampling at any useful temperature does not reach."""
    digest = hashlib.blake2b(struct.pack("<qqq", seed, request_id, token_index), digest_size=8).digest()
    return (int.from_bytes(digest, "little") >> 40) / float(1 << 24)


@dataclass
class Draw:
    """A launched draw: the tokens are on the device (``tokens``) and on their way to the host."""

    tokens: torch.Tensor  # int32 [rows] on the device; the next launch of the sampler overwrites it
    rows: int
    side: int  # which of the two host buffers the tokens arrive in


class Sampler:
    """Draws are launched and collected separately, so that the caller can queue more device work
    (the next step, fed with ``Draw.tokens``) before it waits for the token ids.  At most two draws
    may be outstanding: each launch takes the host buffers that the draw before the last one used."""

    def __init__(self, seed: int, max_rows: int, device: str | torch.device = "cuda"):
        self.seed = seed
        self.device = torch.device(device)
        self._host = torch.empty((2, 2, max_rows), dtype=torch.float32).pin_memory()  # [side][temperature, uniform]
        self._host_np = self._host.numpy()
        self._params = torch.empty((2, 2, max_rows), dtype=torch.float32, device=self.device)
        self._tokens = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._tokens_host = torch.empty((2, max_rows), dtype=torch.int32).pin_memory()
        self._arrived = [torch.cuda.Event(), torch.cuda.Event()]
        self._side = 0

    def launch(
        self,
        logits: torch.Tensor,
        temperatures: Seq[float],
        request_ids: Seq[int],
        token_indices: Seq[int],
    ) -> Draw:
        """Start drawing one token per row of ``logits [rows, vocab]`` (float32, on the device)."""
        rows = logits.shape[0]
        self._side ^= 1
        side = self._side
        out = self._tokens[:rows]
        if rows == 0:
            return Draw(out, 0, side)
        if all(t == 0 for t in temperatures):
            ops.sample(logits, None, None, out)
        else:
            host = self._host_np[side]  # written through numpy: one assignment per row of the block
            host[0, :rows] = temperatures
            host[1, :rows] = [
                uniform_for(self.seed, request_ids[i], token_indices[i]) if temperatures[i] else 0.0 for i in range(rows)
            ]
            params = self._params[side]
            params[:, :rows].copy_(self._host[side][:, :rows], non_blocking=True)
            ops.sample(logits, params[0, :rows], params[1, :rows], out)
        self._tokens_host[side, :rows].copy_(out, non_blocking=True)
        self._arrived[side].record()
        return Draw(out, rows, side)

    def collect(self, draw: Draw) -> list[int]:
        """Wait for a launched draw and return its token ids."""
        if draw.rows == 0:
            return []
        self._arrived[draw.side].synchronize()
        return self._tokens_host[draw.side, : draw.rows].tolist()

    def sample(
        self,
        logits: torch.Tensor,
        temperatures: Seq[float],
        request_ids: Seq[int],
        token_indices: Seq[int],
    ) -> list[int]:
        """One token per row of ``logits [rows, vocab]`` (float32, on the device)."""
        return self.collect(self.launch(logits, temperatures, request_ids, token_indices))
