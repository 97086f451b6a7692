"""A decoder assembled from a :class:`~mini_engine_b200.config.model_spec.ModelSpec`.

The embedding part, the layers in the order that the spec lists, the final norm on the wanted
rows only, then the head part (src/mini_engine/model.py:163-188 of YuvGev00/mini-engine: a
lookup without scaling and a head without bias that may be the embedding matrix itself).
Every one of them is looked up in a registry by the kind its spec names.
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
    build_end,
    build_part,
)
from mini_engine_b200.weights.loader import WeightSpec

# Importing the built-in parts registers them.
from mini_engine_b200.parts import attention, block, ends, mlp, norms, rotary  # noqa: F401,E402


def build_block(spec: ModelSpec, index: int) -> Block:
    """The layer's block with the parts its spec names; the block's class says which norms it
    wants (``Block.NORMS``) and the spec must name exactly those."""
    layer = spec.layers[index]
    if layer.block not in BLOCKS:
        raise KeyError(f"no block named {layer.block!r}; registered: {', '.join(sorted(BLOCKS))}")
    hidden = spec.hidden_size
    norms = {name: build_part("norm", part, layer.prefix, hidden) for name, part in layer.named_norms().items()}
    return BLOCKS[layer.block](
        build_part("mixer", layer.mixer, layer.prefix, hidden),
        build_part("feed_forward", layer.feed_forward, layer.prefix, hidden),
        norms,
    )


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_end("embedding", spec.embedding, spec.vocab_size, spec.hidden_size)
        self.blocks = [build_block(spec, i) for i in range(len(spec.layers))]
        self.final_norm = build_part("norm", spec.final_norm, "", spec.hidden_size)
        self.head = build_end("head", spec.head, spec.vocab_size, spec.hidden_size)

    # ------------------------------------------------------------------ declarations

    def weight_specs(self) -> list[WeightSpec]:
        specs = list(self.embedding.weight_specs())
        for blk in self.blocks:
            specs += blk.weight_specs()
        specs += self.final_norm.weight_specs()
        specs += self.head.weight_specs()
        return specs

    @property
    def capturable(self) -> bool:
        """Whether every part of the model says that a step of a fixed token count may be captured
        in a CUDA graph (see ``Part.capturable``)."""
        parts = [self.embedding, self.final_norm, self.head]
        for blk in self.blocks:
            parts += [blk, *blk.parts()]
            position = getattr(blk.mixer, "position", None)
            if position is not None:
                parts.append(position)
        return all(getattr(part, "capturable", False) for part in parts)

    def cache_needs(self) -> list[tuple[PagedCacheSpec | None, StateSpec | None, int | None]]:
        """For every entry of the execution order: its per-token need, its per-request
        need, and the earlier entry whose cache it reads instead (or ``None``)."""
        needs = []
        for entry in self.spec.order:
            mixer = self.blocks[entry.layer].mixer
            needs.append((mixer.paged_cache(), mixer.state(), entry.cache_of))
        return needs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.embedding.load(tensors)
        for blk in self.blocks:
            blk.load(tensors)
        self.final_norm.load(tensors)
        self.head.load(tensors)

    # ------------------------------------------------------------------------ step

    def forward(self, ctx: StepContext, caches: list[LayerCache], logits_rows: torch.Tensor) -> torch.Tensor:
        """Run the batch's tokens through every entry of the order; return float32 logits
        ``[N, vocab]`` at ``logits_rows`` (int32 row numbers among the batch's tokens)."""
        with ops.stream_scope():
            return self._forward(ctx, caches, logits_rows)

    def _forward(self, ctx: StepContext, caches: list[LayerCache], logits_rows: torch.Tensor) -> torch.Tensor:
        x = ctx.buffer("residual", (ctx.num_tokens, self.spec.hidden_size), torch.float32)
        self.embedding.forward(ctx.token_ids, ctx, x)
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
        return self.head.forward(rows, ctx)


def declared_weights(spec: ModelSpec) -> list[WeightSpec]:
    """Every tensor that the model of ``spec`` reads from a checkpoint (no GPU needed)."""
    return DecoderModel(spec).weight_specs()
