"""Arrangements of a layer's parts around the residual stream."""

from __future__ import annotations

from mini_engine_b200.parts.base import Block, LayerCache, Residual, StepContext, register


@register("block", "prenorm")
class PreNormBlock(Block):
    """``h = x + mixer(norm(x))``, ``y = h + feed_forward(norm(h))``
    (src/mini_engine/model.py:149-150 of YuvGev00/mini-engine).  The two sums happen inside
    the norms that follow them (the last one inside the next layer's first norm or the
    model's final norm), in 32-bit."""

    capturable = True

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        h = self.mixer_norm.forward(state, ctx, ctx.dtype)
        state.add(self.mixer.forward(h, ctx, cache))
        h = self.feed_forward_norm.forward(state, ctx, ctx.dtype)
        state.add(self.feed_forward.forward(h, ctx))
