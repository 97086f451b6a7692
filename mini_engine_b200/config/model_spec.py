"""The model as data: which parts each layer is made of, and in which order layers run.

An architecture turns its typed configuration into a :class:`ModelSpec`.  Nothing below
the architecture module knows a model's name: parts are looked up by ``PartSpec.kind`` in
the part registries and receive ``PartSpec.params`` as their constants.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registry key of its implementation and its constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One set of layer weights.

    ``prefix`` is the checkpoint name prefix of the layer's tensors (for example
    ``model.layers.3.``).  ``block`` names the arrangement of the parts (for example pre-norm
    residual).  Different layers may name different mixers and feed-forwards.  ``norms`` maps the
    names that the block's class asks for to norm parts: a pre-norm block asks for ``"mixer"``
    and ``"feed_forward"`` (the norm in front of each); another arrangement may ask for more
    (norms behind the mixer and the feed-forward, say).  ``mixer_norm`` and
    ``feed_forward_norm`` are those two entries under their old names.
    """

    prefix: str
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec | None = None
    feed_forward_norm: PartSpec | None = None
    norms: Mapping[str, PartSpec] = field(default_factory=dict)

    def named_norms(self) -> dict[str, PartSpec]:
        """Every norm of the layer by the name its block knows it under."""
        named = dict(self.norms)
        for name, spec in (("mixer", self.mixer_norm), ("feed_forward", self.feed_forward_norm)):
            if spec is not None:
                if name in named:
                    raise ValueError(f"layer {self.prefix!r} names its {name!r} norm twice")
                named[name] = spec
        return named


@dataclass(frozen=True)
class OrderEntry:
    """One execution of a layer.

    ``layer`` indexes :attr:`ModelSpec.layers`; the same index may appear in several
    entries (the weights are then shared, each entry keeps a cache of its own).
    ``cache_of`` is ``None`` when the entry owns its cache, else the index of an *earlier
    entry* whose cache this entry's mixer reads without writing to it.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[OrderEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def __post_init__(self) -> None:
        for position, entry in enumerate(self.order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"order[{position}] names layer {entry.layer}, which does not exist")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < position:
                    raise ValueError(
                        f"order[{position}] reads the cache of entry {entry.cache_of}; "
                        "it must be an earlier entry"
                    )
                if self.order[entry.cache_of].cache_of is not None:
                    raise ValueError(f"order[{position}] must read the cache of an entry that owns one")
