"""The two ends of a model as parts: token embedding and output head.

``token_embedding``: ``x = E[token_ids]``, times ``multiplier`` when the model scales its
embeddings (the reference's decoder does not: src/mini_engine/model.py:182 of
YuvGev00/mini-engine).  ``linear_head``: ``logits = rows W^T`` without bias, where ``W`` may be
the embedding matrix itself (``tied_to``; src/mini_engine/model.py:168-170,186-187); a head may
also have a bias, a logit scale and a soft cap ``cap * tanh(logits / cap)``, applied in that
order by one small kernel.  Both are looked up by ``PartSpec.kind`` like every other part, so a
model with another first or last part registers its own and changes nothing here.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import Embedding, Head, StepContext, register
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, *, weight: str, multiplier: float | None = None):
        self.vocab, self.hidden = vocab_size, hidden_size
        self.weight_name = weight
        self.multiplier = 1.0 if multiplier is None else float(multiplier)
        self.table: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.vocab, self.hidden))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.weight_name]

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, out: torch.Tensor) -> None:
        ops.embedding(self.table, token_ids, out, self.multiplier)


@register("head", "linear_head")
class LinearHead(Head):
    capturable = True

    def __init__(
        self,
        vocab_size: int,
        hidden_size: int,
        *,
        weight: str,
        tied_to: str | None = None,
        bias: str | None = None,
        logit_scale: float | None = None,
        soft_cap: float | None = None,
    ):
        self.vocab, self.hidden = vocab_size, hidden_size
        self.weight_name, self.tied_to, self.bias_name = weight, tied_to, bias
        self.logit_scale = 1.0 if logit_scale is None else float(logit_scale)
        self.soft_cap = 0.0 if soft_cap is None else float(soft_cap)
        if self.soft_cap < 0:
            raise ValueError("soft_cap must be positive (or absent)")
        self.linear: Linear | None = None
        self.bias: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        specs = [WeightSpec(self.weight_name, (self.vocab, self.hidden), alias_of=self.tied_to)]
        if self.bias_name:
            specs.append(WeightSpec(self.bias_name, (self.vocab,), role="vector"))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.linear = Linear(tensors[self.weight_name])
        self.bias = tensors[self.bias_name] if self.bias_name else None

    def forward(self, rows: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = self.linear.forward(rows, ctx, "logits", whole=True)[0]
        if self.bias is not None or self.logit_scale != 1.0 or self.soft_cap > 0.0:
            ops.logits_finish(logits, self.bias, self.logit_scale, self.soft_cap)
        return logits
