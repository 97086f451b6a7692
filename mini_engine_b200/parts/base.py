"""Interfaces and registries of the parts a layer is made of.

A layer is assembled from parts and an arrangement:

* a **mixer** (token mixing: attention here) that may keep per-token pages and/or a
  fixed-size per-request state in the cache manager,
* a **feed-forward**,
* **norms**, by the names that the arrangement asks for (two in a pre-norm layer),
* a **block** that says how they are wired (pre-norm residual here),

and a mixer may own a **position encoding**.  The model's two ends are parts as well: an
**embedding** and a **head**.  Each kind has one registry from a name to a
class; a :class:`~mini_engine_b200.config.model_spec.PartSpec` names the class and carries
its constants.  No part reads a model configuration or knows which model it is in.

The hidden state travels as a :class:`Residual`: the 32-bit residual stream plus the
not-yet-added output of the previous part.  A norm adds the pending output while it
normalises, which fuses the residual sum (in 32-bit) with the next norm's read.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch

from mini_engine_b200.config.model_spec import PartSpec
from mini_engine_b200.weights.loader import WeightSpec

# ------------------------------------------------------------------------------ cache needs


@dataclass(frozen=True)
class PagedCacheSpec:
    """Per-token cache of one mixer: K and V of ``kv_heads`` heads of ``head_dim`` values.

    ``window`` is ``None`` when every key is kept; else only the last ``window`` positions
    are ever read and pages wholly behind the window are given back while the request runs.
    Mixers with an equal spec share one cache group (one page pool, one block table per
    request).
    """

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: ``shape`` elements of ``dtype`` per request."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------------------- step-time data


@dataclass
class Residual:
    """The residual stream ``x [T, hidden]`` (float32) and a pending addend.

    ``pending`` is ``None`` or a float32 tensor ``[S, T, hidden]`` whose ``S`` slices (the
    partial sums of a split matrix product) are all still to be added to ``x``.
    """

    x: torch.Tensor
    pending: torch.Tensor | None = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            raise RuntimeError("a pending output must be consumed by a norm before the next is set")
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        self.pending = delta


@dataclass
class LayerCache:
    """What one execution of a mixer sees of the cache.

    ``k`` and ``v`` are the page arrays of this entry, ``[pages + 1, kv_heads, page_size,
    head_dim]`` (the last page is a spare that no request owns); ``group`` indexes the
    per-group arrays of :class:`StepContext`; ``writes`` is False when the entry reads
    another entry's cache.  ``state`` is ``[slots + 1, *StateSpec.shape]`` or ``None``.
    """

    group: int | None = None
    k: torch.Tensor | None = None
    v: torch.Tensor | None = None
    writes: bool = True
    state: torch.Tensor | None = None


@dataclass
class StepContext:
    """One batch of (request, its next tokens), flattened; all index tensors are int32.

    Tokens of all entries are concatenated in entry order.  Entry ``b`` owns tokens
    ``cu_tokens[b] .. cu_tokens[b+1]``, which are the positions ``context_lens[b] - n_b ..
    context_lens[b] - 1`` of its request.
    """

    dtype: torch.dtype  # compute dtype of matrices and activations
    num_tokens: int
    num_entries: int
    max_query_len: int
    max_context_len: int
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T] absolute position of each token in its request
    entry_of_token: torch.Tensor  # [T]
    cu_tokens: torch.Tensor  # [B + 1]
    context_lens: torch.Tensor  # [B] tokens of the request after this step
    state_slots: torch.Tensor  # [B] slot of the request's fixed-size state
    fresh: torch.Tensor  # [B] 1 when the entry starts at position 0 (state starts from zero)
    slot_mapping: list[torch.Tensor] = field(default_factory=list)  # per group [T]: page * page_size + offset
    block_tables: list[torch.Tensor] = field(default_factory=list)  # per group [B, max_blocks]
    page_size: int = 16
    workspace: "Any" = None  # Workspace: named persistent buffers
    all_decode: bool = False  # every entry brings exactly one token
    num_decode_entries: int = 0  # entries that bring exactly one token ...
    decode_entries: torch.Tensor | None = None  # ... their numbers, ascending (int32)
    portion_entries: torch.Tensor | None = None  # the numbers of the entries that bring more
    host: Mapping[str, Any] = field(default_factory=dict)  # host copies for parts written in Python
    memo: dict = field(default_factory=dict)  # what parts compute once per step and share between layers

    def buffer(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype)


# ------------------------------------------------------------------------------ interfaces


class Part:
    """Common to all parts: declared weights and their arrival."""

    # Whether the part's launches depend on the batch through device arrays and the token count
    # alone, so that a step of a fixed token count can be captured in a CUDA graph and replayed for
    # other requests (a part whose Python reads ``ctx.host`` or branches on values must say False).
    capturable = False

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the declared tensors (already on the device, cast by role)."""


class Norm(Part):
    def forward(
        self, state: Residual, ctx: StepContext, out_dtype: torch.dtype, rows: torch.Tensor | None = None
    ) -> torch.Tensor:
        """Add ``state.pending`` into ``state.x`` (and clear it), return the normalised rows
        in ``out_dtype``.  With ``rows`` (int32 ``[N]``) only those rows are produced, as
        ``[N, hidden]``, and ``state.x`` is left as it was."""
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_rotary_table(self) -> torch.Tensor | None:
        """Inverse frequencies ``[rotary_dim / 2]`` (float32, on the device) when the
        encoding is a rotate-half rotation that the mixer's fused kernel can apply; else
        ``None`` and the mixer calls :meth:`apply`."""
        return None

    def step_angles(self, ctx: "StepContext") -> torch.Tensor | None:
        """``[T, rotary_dim / 2, 2]`` float32 (cos, sin) for the step's tokens when the
        encoding is a fusable rotation, made once per step and shared by all layers."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode positions in place into ``q [T, heads, d]`` and ``k [T, kv_heads, d]``.
        Keys are cached after this call, so the encoding may depend on the absolute
        position only."""
        raise NotImplementedError


class Mixer(Part):
    def paged_cache(self) -> PagedCacheSpec | None:
        return None

    def state(self) -> StateSpec | None:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """``h [T, hidden]`` (compute dtype) -> output ``[S, T, hidden]`` float32 whose ``S``
        slices sum to the mixer's output."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """``h [T, hidden]`` -> ``[S, T, hidden]`` float32, as for a mixer."""
        raise NotImplementedError


class Embedding(Part):
    """The model's first part: token ids to rows of the residual stream."""

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, out: torch.Tensor) -> None:
        """Fill ``out [T, hidden]`` (float32, the residual stream) for ``token_ids [T]`` (int32)."""
        raise NotImplementedError


class Head(Part):
    """The model's last part: normalised rows to logits."""

    def forward(self, rows: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """``rows [N, hidden]`` (compute dtype) -> float32 logits ``[N, vocab]``."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of mixer, feed-forward and norms around the residual stream.

    ``NORMS`` lists the names of the norms that the arrangement uses; the layer's spec must give
    exactly those (``LayerSpec.named_norms``), and they arrive as ``self.norms[name]``."""

    NORMS: tuple[str, ...] = ("mixer", "feed_forward")

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Mapping[str, Norm]):
        if set(norms) != set(self.NORMS):
            raise ValueError(
                f"{type(self).__name__} wants the norms {sorted(self.NORMS)}, the layer names {sorted(norms)}"
            )
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)

    @property
    def mixer_norm(self) -> Norm:
        return self.norms["mixer"]

    @property
    def feed_forward_norm(self) -> Norm:
        return self.norms["feed_forward"]

    def parts(self) -> list[Part]:
        return [self.mixer, self.feed_forward, *(self.norms[name] for name in self.NORMS)]

    def weight_specs(self) -> list[WeightSpec]:
        return [spec for part in self.parts() for spec in part.weight_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        raise NotImplementedError


# ------------------------------------------------------------------------------ registries

Factory = Callable[..., Any]

MIXERS: dict[str, Factory] = {}
FEED_FORWARDS: dict[str, Factory] = {}
NORMS: dict[str, Factory] = {}
POSITION_ENCODINGS: dict[str, Factory] = {}
BLOCKS: dict[str, Factory] = {}
EMBEDDINGS: dict[str, Factory] = {}
HEADS: dict[str, Factory] = {}

_REGISTRIES = {
    "mixer": MIXERS,
    "feed_forward": FEED_FORWARDS,
    "norm": NORMS,
    "position_encoding": POSITION_ENCODINGS,
    "block": BLOCKS,
    "embedding": EMBEDDINGS,
    "head": HEADS,
}


def register(kind: str, name: str, replace: bool = False) -> Callable[[Factory], Factory]:
    """Class decorator: ``@register("mixer", "gqa_attention")``.

    A mixer, feed-forward, norm or position encoding is built as ``cls(prefix, hidden_size,
    **PartSpec.params)`` where ``prefix`` is the checkpoint prefix of the layer; a block as
    ``cls(mixer, feed_forward, norms)`` with ``norms`` a mapping from the names in its ``NORMS``
    to norm parts; an embedding or a head as ``cls(vocab_size, hidden_size, **PartSpec.params)``.
    """
    registry = _REGISTRIES[kind]

    def decorate(cls: Factory) -> Factory:
        if name in registry and not replace:
            raise ValueError(f"{kind} {name!r} is already registered")
        registry[name] = cls
        return cls

    return decorate


def build_end(kind: str, spec: PartSpec, vocab_size: int, hidden_size: int) -> Any:
    """An ``"embedding"`` or a ``"head"``: ``cls(vocab_size, hidden_size, **PartSpec.params)``."""
    registry = _REGISTRIES[kind]
    if spec.kind not in registry:
        raise KeyError(f"no {kind} named {spec.kind!r}; registered: {', '.join(sorted(registry))}")
    return registry[spec.kind](vocab_size, hidden_size, **dict(spec.params))


def build_part(kind: str, spec: PartSpec, prefix: str, hidden_size: int) -> Any:
    registry = _REGISTRIES[kind]
    if spec.kind not in registry:
        raise KeyError(f"no {kind} named {spec.kind!r}; registered: {', '.join(sorted(registry))}")
    return registry[spec.kind](prefix, hidden_size, **dict(spec.params))
