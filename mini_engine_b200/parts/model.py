"""A decoder assembled from a :class:`~mini_engine_b200.config.model_spec.ModelSpec`.

Embedding lookup without scaling, the layers in the order that the spec lists, the final
norm on the wanted rows only, then the head without bias; the head may be the embedding
matrix itself (src/mini_engine/model.py:163-188 of YuvGev00/mini-engine).
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.config.model_spec import ModelSpec
from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import (
    BLOCKS,
    Block,
    LayerCache,
    PagedCacheSpec,
    Residual,
    StateSpec,
    StepContext,
    build_part,
)
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec

# Importing the built-in parts registers them.
from mini_engine_b200.parts import attention, block, mlp, norms, rotary  # noqa: F401,E402


def build_block(spec: ModelSpec, index: int) -> Block:
    layer = spec.layers[index]
    if layer.block not in BLOCKS:
        raise KeyError(f"no block named {layer.block!r}; registered: {', '.join(sorted(BLOCKS))}")
    hidden = spec.hidden_size
    return BLOCKS[layer.block](
        build_part("mixer", layer.mixer, layer.prefix, hidden),
        build_part("feed_forward", layer.feed_forward, layer.prefix, hidden),
        build_part("norm", layer.mixer_norm, layer.prefix, hidden),
        build_part("norm", layer.feed_forward_norm, layer.prefix, hidden),
    )


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks = [build_block(spec, i) for i in range(len(spec.layers))]
        self.final_norm = build_part("norm", spec.final_norm, "", spec.hidden_size)
        self.embedding_name: str = spec.embedding["weight"]
        self.head_name: str = spec.head["weight"]
        self.head_tied_to: str | None = spec.head.get("tied_to")
        self.embedding: torch.Tensor | None = None
        self.head: Linear | None = None

    # ------------------------------------------------------------------ declarations

    def weight_specs(self) -> list[WeightSpec]:
        shape = (self.spec.vocab_size, self.spec.hidden_size)
        specs = [WeightSpec(self.embedding_name, shape)]
        for blk in self.blocks:
            specs += blk.weight_specs()
        specs += self.final_norm.weight_specs()
        specs.append(WeightSpec(self.head_name, shape, alias_of=self.head_tied_to))
        return specs

    def cache_needs(self) -> list[tuple[PagedCacheSpec | None, StateSpec | None, int | None]]:
        """For every entry of the execution order: its per-token need, its per-request
        need, and the earlier entry whose cache it reads instead (or ``None``)."""
        needs = []
        for entry in self.spec.order:
            mixer = self.blocks[entry.layer].mixer
            needs.append((mixer.paged_cache(), mixer.state(), entry.cache_of))
        return needs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.embedding = tensors[self.embedding_name]
        for blk in self.blocks:
            blk.load(tensors)
        self.final_norm.load(tensors)
        self.head = Linear(tensors[self.head_name])

    # ------------------------------------------------------------------------ step

    def forward(self, ctx: StepContext, caches: list[LayerCache], logits_rows: torch.Tensor) -> torch.Tensor:
        """Run the batch's tokens through every entry of the order; return float32 logits
        ``[N, vocab]`` at ``logits_rows`` (int32 row numbers among the batch's tokens)."""
        with ops.stream_scope():
            return self._forward(ctx, caches, logits_rows)

    def _forward(self, ctx: StepContext, caches: list[LayerCache], logits_rows: torch.Tensor) -> torch.Tensor:
        x = ctx.buffer("residual", (ctx.num_tokens, self.spec.hidden_size), torch.float32)
        ops.embedding(self.embedding, ctx.token_ids, x)
        state = Residual(x)
        for entry, cache in zip(self.spec.order, caches, strict=True):
            self.blocks[entry.layer].forward(state, ctx, cache)
        count = logits_rows.shape[0]
        if count == 0:
            # Nothing is wanted, but the last pending sum must not be left on the state.
            state.pending = None
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        rows = self.final_norm.forward(state, ctx, ctx.dtype, rows=logits_rows)
        state.pending = None
        return self.head.forward(rows, ctx, "logits", whole=True)[0]


def declared_weights(spec: ModelSpec) -> list[WeightSpec]:
    """Every tensor that the model of ``spec`` reads from a checkpoint (no GPU needed)."""
    return DecoderModel(spec).weight_specs()
