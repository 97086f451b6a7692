"""Dense gated feed-forward (SwiGLU) as a part.

``y = (silu(x Wg^T) * (x Wu^T)) Wd^T`` with ``silu(a) = a * sigmoid(a)`` and no biases
(src/mini_engine/model.py:122-131 of YuvGev00/mini-engine).  Gate and up run as one product
on the row-concatenated weight; on the tensor-core path the activation is applied in that
product's epilogue, so the ``[T, 2 * inter]`` intermediate never reaches memory.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.parts.base import FeedForward, StepContext, register
from mini_engine_b200.parts.linear import GatedLinear, Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    capturable = True

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        intermediate_size: int,
        activation: str = "silu",
        names: Mapping[str, str] | None = None,
    ):
        if activation != "silu":
            raise ValueError(f"gated_mlp implements the 'silu' gate only, got {activation!r}")
        self.hidden, self.inter = hidden_size, intermediate_size
        defaults = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        self.gate_up: GatedLinear | None = None
        self.down: Linear | None = None

    def weight_specs(self) -> list[WeightSpec]:
        n = self.names
        return [
            WeightSpec(n["gate"], (self.inter, self.hidden)),
            WeightSpec(n["up"], (self.inter, self.hidden)),
            WeightSpec(n["down"], (self.hidden, self.inter)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.gate_up = GatedLinear(torch.cat((tensors[n["gate"]], tensors[n["up"]]), dim=0).contiguous())
        self.down = Linear(tensors[n["down"]])

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = self.gate_up.forward(h, ctx, "mlp")
        return self.down.forward(act, ctx, "mlp.down")
