"""Grouped-query attention over the paged cache, as a mixer part.

Formulas (YuvGev00/mini-engine): ``q, k, v = x Wq^T, x Wk^T, x Wv^T`` without biases, q and k
normalised per head with one weight ``[head_dim]`` shared by all heads, then rotated, in
that order (src/mini_engine/model.py:97-118); new keys and values are written to the cache
first, then every query reads all its keys from the cache (src/mini_engine/attention.py:117-121);
query head ``h`` reads KV head ``h // (heads / kv_heads)``, scores are scaled by
``head_dim**-0.5``, the query at position ``p`` sees positions ``<= p``
(src/mini_engine/attention.py:84-86,160-175).

The three projections run as one product on the row-concatenated weight, which leaves every
output element's sum unchanged.  Per-head norm, rotation and the cache write are one kernel.
All sizes and constants are constructor arguments; the part does not know its model.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from mini_engine_b200.config.model_spec import PartSpec
from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import (
    LayerCache,
    Mixer,
    PagedCacheSpec,
    StepContext,
    build_part,
    register,
)
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("mixer", "gqa_attention")
class GroupedQueryAttention(Mixer):
    capturable = True

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        num_heads: int,
        kv_heads: int,
        head_dim: int,
        position_encoding: PartSpec,
        qk_norm_eps: float | None = None,
        window: int | None = None,
        scale: float | None = None,
        reads_shared_cache: bool = False,
        qkv_bias: bool = False,
        names: Mapping[str, str] | None = None,
    ):
        if num_heads % kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of kv_heads ({kv_heads})")
        ops.check_attention_sizes(head_dim, num_heads, kv_heads)
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden_size, num_heads, kv_heads, head_dim
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else head_dim**-0.5
        self.reads_shared_cache = reads_shared_cache
        self.qkv_bias = qkv_bias  # the reference's projections have none (src/mini_engine/model.py:97-100)
        defaults = {
            "q": "q_proj.weight",
            "k": "k_proj.weight",
            "v": "v_proj.weight",
            "o": "o_proj.weight",
            "q_norm": "q_norm.weight",
            "k_norm": "k_norm.weight",
            "q_bias": "q_proj.bias",
            "k_bias": "k_proj.bias",
            "v_bias": "v_proj.bias",
        }
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        self.position = build_part("position_encoding", position_encoding, prefix, hidden_size)
        self.qkv: Linear | None = None
        self.out: Linear | None = None
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    # ------------------------------------------------------------------ declarations

    def paged_cache(self) -> PagedCacheSpec:
        return PagedCacheSpec(self.kv_heads, self.head_dim, self.window)

    def weight_specs(self) -> list[WeightSpec]:
        d, n = self.head_dim, self.names
        specs = [WeightSpec(n["q"], (self.heads * d, self.hidden))]
        if not self.reads_shared_cache:
            specs += [
                WeightSpec(n["k"], (self.kv_heads * d, self.hidden)),
                WeightSpec(n["v"], (self.kv_heads * d, self.hidden)),
            ]
        specs.append(WeightSpec(n["o"], (self.hidden, self.heads * d)))
        if self.qk_norm_eps is not None:
            specs.append(WeightSpec(n["q_norm"], (d,), role="vector", init="ones_normal"))
            if not self.reads_shared_cache:
                specs.append(WeightSpec(n["k_norm"], (d,), role="vector", init="ones_normal"))
        if self.qkv_bias:
            specs.append(WeightSpec(n["q_bias"], (self.heads * d,), role="vector"))
            if not self.reads_shared_cache:
                specs.append(WeightSpec(n["k_bias"], (self.kv_heads * d,), role="vector"))
                specs.append(WeightSpec(n["v_bias"], (self.kv_heads * d,), role="vector"))
        return specs + self.position.weight_specs()

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [tensors[n["q"]]]
        if not self.reads_shared_cache:
            rows += [tensors[n["k"]], tensors[n["v"]]]
        self.qkv = Linear(torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0])
        self.out = Linear(tensors[n["o"]])
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[n["q_norm"]]
            self.k_norm = None if self.reads_shared_cache else tensors[n["k_norm"]]
        if self.qkv_bias:
            parts = [tensors[n["q_bias"]]]
            if not self.reads_shared_cache:
                parts += [tensors[n["k_bias"]], tensors[n["v_bias"]]]
            self.bias = torch.cat(parts).contiguous()
        self.position.load(tensors)

    # ------------------------------------------------------------------------ step

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        tokens, d = h.shape[0], self.head_dim
        kv_in = 0 if self.reads_shared_cache else self.kv_heads
        qkv = self.qkv.forward(h, ctx, "attn.qkv")
        q = ctx.buffer("attn.q", (tokens, self.heads * d), ctx.dtype)
        table = self.position.step_angles(ctx)
        slots = ctx.slot_mapping[cache.group]
        args: dict[str, Any] = dict(
            qkv=qkv, heads=self.heads, kv_heads=kv_in, head_dim=d, q_weight=self.q_norm,
            k_weight=self.k_norm, eps=self.qk_norm_eps or 0.0, positions=ctx.positions, q_out=q,
            page_size=ctx.page_size, bias=self.bias,
        )  # fmt: skip
        if kv_in and not cache.writes:
            # This execution reads another entry's cache: its own keys and values are not kept.
            unused_k = ctx.buffer("attn.k_new", (tokens, kv_in * d), ctx.dtype)
            unused_v = ctx.buffer("attn.v_new", (tokens, kv_in * d), ctx.dtype)
            ops.qk_norm_rope_store(**args, cos_sin=table, k_dense=unused_k, v_dense=unused_v)
            if table is None:
                self.position.apply(q.view(tokens, self.heads, d), unused_k.view(tokens, kv_in, d), ctx.positions)
        elif table is not None or kv_in == 0:
            ops.qk_norm_rope_store(
                **args, cos_sin=table, slot_mapping=slots, k_pages=cache.k, v_pages=cache.v
            )
        else:  # a position encoding that the fused kernel does not know: three steps
            k_new = ctx.buffer("attn.k_new", (tokens, kv_in * d), ctx.dtype)
            v_new = ctx.buffer("attn.v_new", (tokens, kv_in * d), ctx.dtype)
            ops.qk_norm_rope_store(**args, cos_sin=None, k_dense=k_new, v_dense=v_new)
            self.position.apply(q.view(tokens, self.heads, d), k_new.view(tokens, kv_in, d), ctx.positions)
            ops.kv_store(k_new, v_new, slots, cache.k, cache.v, kv_in, d, ctx.page_size)
        out = ctx.buffer("attn.out", (tokens, self.heads * d), ctx.dtype)
        ops.paged_attention(
            q=q, k_pages=cache.k, v_pages=cache.v, block_table=ctx.block_tables[cache.group], ctx=ctx,
            out=out, heads=self.heads, kv_heads=self.kv_heads, head_dim=d, scale=self.scale,
            window=self.window or 0,
        )  # fmt: skip
        return self.out.forward(out, ctx, "attn.o")
