"""RMSNorm as a part.

``y = w * (x * rsqrt(mean(x^2) + eps))`` with the statistics in 32-bit, eps inside the root
(src/mini_engine/model.py:59-69 of YuvGev00/mini-engine).  The reference rounds the
normalised value to the model dtype before the weight multiply; here the whole expression
is evaluated in 32-bit and rounded once, which is at least as accurate.  The norm also
performs the residual sum that precedes it (see :class:`~mini_engine_b200.parts.base.Residual`).
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import Norm, Residual, StepContext, register
from mini_engine_b200.weights.loader import WeightSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    capturable = True

    def __init__(self, prefix: str, hidden_size: int, *, name: str, eps: float, dim: int | None = None):
        self.weight_name = prefix + name
        self.dim = dim or hidden_size
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.dim,), role="vector", init="ones_normal")]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]

    def forward(self, state: Residual, ctx: StepContext, out_dtype, rows=None) -> torch.Tensor:
        count = state.x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer("norm.out" if rows is None else "norm.rows", (count, self.dim), out_dtype)
        ops.add_rmsnorm(state.x, state.pending, self.weight, self.eps, out, rows)
        if rows is None:
            state.pending = None
        return out
