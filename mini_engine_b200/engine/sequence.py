"""One request as the engine tracks it.

The attribute names are those of YuvGev00/mini-engine's ``Sequence``
(src/mini_engine/sequence.py:23-77), because callers and the scheduler's policy are written
against them: ``token_ids`` (prompt and generated ids in one list), ``num_computed_tokens``,
``num_prompt_tokens``, ``num_cached_tokens``, ``num_preemptions``, ``status`` and the derived
counts.  What a request holds in the cache is not kept here as lists of pages and hashes but in
one :class:`~mini_engine_b200.cache.manager.RequestCache` (a block table per cache group, the page
hashes, the state slot), which the cache manager owns.

The invariant everything rests on: the tokens ``[0, num_computed_tokens)`` have left what they
leave behind in the cache (keys and values in the pages of ``cache.block_tables``, per-request
state in ``cache.state_slot``), and the scheduler only ever asks for the tokens
``[num_computed_tokens, len(token_ids))``.  A whole prompt, a portion of one, a single decoded
token and the recomputation after a preemption are therefore the same operation.
"""

from __future__ import annotations

import enum
import itertools
from typing import Iterable

from mini_engine_b200.cache.manager import RequestCache
from mini_engine_b200.sampling.params import SamplingParams


class SequenceStatus(enum.Enum):
    WAITING = enum.auto()
    RUNNING = enum.auto()
    FINISHED = enum.auto()


_next_id = itertools.count()


class Sequence:
    """A request from submission to its last token.  ``seq_id`` seeds the request's sampling
    stream together with the engine's seed, so a caller that wants the same draws again passes
    the same id."""

    __slots__ = (
        "token_ids", "params", "seq_id", "status", "num_prompt_tokens", "num_computed_tokens",
        "num_cached_tokens", "num_preemptions", "cache",
    )  # fmt: skip

    def __init__(self, token_ids: Iterable[int], params: SamplingParams | None = None, seq_id: int | None = None):
        self.token_ids: list[int] = [int(token) for token in token_ids]
        if not self.token_ids:
            raise ValueError("prompt must contain at least one token")
        self.params = params if params is not None else SamplingParams()
        self.seq_id = next(_next_id) if seq_id is None else int(seq_id)
        self.status = SequenceStatus.WAITING
        self.num_prompt_tokens = len(self.token_ids)
        self.num_computed_tokens = 0
        self.num_cached_tokens = 0  # tokens that the prefix cache served at the last admission
        self.num_preemptions = 0
        self.cache: RequestCache | None = None  # given by the scheduler on submission

    def __len__(self) -> int:
        return len(self.token_ids)

    def __repr__(self) -> str:
        return (
            f"Sequence(id={self.seq_id}, {self.status.name.lower()}, prompt={self.num_prompt_tokens}, "
            f"generated={self.num_output_tokens}, computed={self.num_computed_tokens})"
        )

    # ------------------------------------------------------------------ derived counts

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_uncomputed_tokens(self) -> int:
        return len(self.token_ids) - self.num_computed_tokens

    @property
    def output_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens :]

    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    @property
    def block_table(self) -> list[int]:
        """Pages of the first cache group (the only one of a model whose layers all keep every
        key); empty before admission."""
        if self.cache is None or not self.cache.block_tables:
            return []
        return self.cache.block_tables[0]
