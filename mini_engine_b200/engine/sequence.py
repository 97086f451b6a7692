"""One request's state (src/mini_engine/sequence.py:23-77 of YuvGev00/mini-engine).

Invariant: tokens ``[0, num_computed_tokens)`` have what they leave behind in the cache, in
the pages that ``cache.block_tables`` list.  The scheduler only ever asks for tokens
``[num_computed_tokens, len(token_ids))``, so a prompt, a portion of a prompt, a decoded
token and a recomputation after preemption are the same operation.
"""

from __future__ import annotations

import enum
import itertools
from dataclasses import dataclass, field

from mini_engine_b200.cache.manager import RequestCache
from mini_engine_b200.sampling.params import SamplingParams


class SequenceStatus(enum.Enum):
    WAITING = enum.auto()
    RUNNING = enum.auto()
    FINISHED = enum.auto()


_ids = itertools.count()


@dataclass(eq=False)
class Sequence:
    token_ids: list[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    seq_id: int = field(default_factory=lambda: next(_ids))
    status: SequenceStatus = SequenceStatus.WAITING
    num_computed_tokens: int = 0
    cache: RequestCache | None = None  # set by the scheduler on submission
    num_prompt_tokens: int = field(init=False)
    num_cached_tokens: int = 0  # tokens served by the prefix cache at the last admission
    num_preemptions: int = 0

    def __post_init__(self) -> None:
        if not self.token_ids:
            raise ValueError("prompt must contain at least one token")
        self.token_ids = [int(t) for t in self.token_ids]
        self.num_prompt_tokens = len(self.token_ids)

    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def block_table(self) -> list[int]:
        """Pages of the first cache group (the only one of a model whose layers all keep
        every key)."""
        return self.cache.block_tables[0] if self.cache and self.cache.block_tables else []

    @property
    def num_uncomputed_tokens(self) -> int:
        return len(self.token_ids) - self.num_computed_tokens

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def output_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens :]

    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED
