"""What a step is made of: entries of (request, its next tokens).

A :class:`StepEntry` is the unit that the step function takes (``ModelRunner.execute``), that the
scheduler emits and that the replay program builds from a trace: tokens ``[start, start +
len(token_ids))`` of one request and the places among them whose logits are wanted.  It is plain
host data, so the scheduler needs nothing of the device to make one.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence as Seq

from mini_engine_b200.cache.manager import RequestCache


@dataclass
class StepEntry:
    """Tokens ``[start, start + len(token_ids))`` of one request."""

    cache: RequestCache
    start: int
    token_ids: Seq[int]
    want: Seq[int] = field(default_factory=tuple)  # places among these tokens whose logits are returned
