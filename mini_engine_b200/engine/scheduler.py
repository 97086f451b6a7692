"""Continuous batching under a token budget, with portions of prompts and recompute
preemption (src/mini_engine/scheduler.py:44-159 of YuvGev00/mini-engine).

Every step builds one batch.  A scheduled request brings ``n`` tokens starting at its
``num_computed_tokens``: one for a decode, more for a prompt or a portion of one.

Policy, first come first served:

1. Running requests first, in admission order, each taking ``min(uncomputed, budget)``
   tokens.  **When pages run out**, the most recently admitted running request is
   preempted: everything it holds is given back, its tokens (generated ones included) are
   kept, its computed count returns to zero and it goes to the *front* of the waiting
   queue; this repeats until the allocation succeeds or the request that needs the pages
   is itself the victim.  Victims come from the tail, which the loop has not reached, so a
   victim is never already in the batch.
2. Then waiting requests are admitted in order, reusing cached prefix pages, until the
   budget, the request cap or the pages run out.  Admission stops at the first request
   that does not fit (nobody jumps the queue) and is skipped entirely in a step that
   preempted.

Pure host code: no tensors.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass

from mini_engine_b200.cache.manager import CacheManager
from mini_engine_b200.engine.sequence import Sequence, SequenceStatus


@dataclass(frozen=True)
class SchedulerConfig:
    max_num_seqs: int = 16
    max_num_batched_tokens: int = 2048
    max_model_len: int = 4096


@dataclass
class ScheduledSeq:
    seq: Sequence
    num_tokens: int

    @property
    def samples(self) -> bool:
        """Whether this step reaches the end of the request, so that its logits are used."""
        return self.seq.num_computed_tokens + self.num_tokens == len(self.seq)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager, eos_token_ids: set[int]):
        self.config = config
        self.cache = cache
        self.eos_token_ids = set(eos_token_ids)
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0
        self.num_cached_tokens = 0  # tokens served by the prefix cache, over all admissions

    def add(self, seq: Sequence) -> None:
        longest = len(seq) + seq.params.max_tokens
        if longest > self.config.max_model_len:
            raise ValueError(f"prompt + max_tokens = {longest} exceeds max_model_len {self.config.max_model_len}")
        if self.cache.blocks_needed(longest) > self.cache.num_blocks:
            raise ValueError(f"request needs more than the {self.cache.num_blocks} KV blocks available")
        seq.cache = self.cache.new_request()
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def schedule(self) -> list[ScheduledSeq]:
        budget = self.config.max_num_batched_tokens
        batch: list[ScheduledSeq] = []
        preempted = False

        index = 0
        while index < len(self.running) and budget > 0:
            seq = self.running[index]
            count = min(seq.num_uncomputed_tokens, budget)
            granted = self.cache.try_allocate(seq.cache, seq.num_computed_tokens + count)
            while not granted:
                victim = self.running[-1]
                self._preempt(victim)
                preempted = True
                if victim is seq:
                    break
                granted = self.cache.try_allocate(seq.cache, seq.num_computed_tokens + count)
            if granted:
                batch.append(ScheduledSeq(seq, count))
                budget -= count
                index += 1

        while (
            not preempted
            and self.waiting
            and budget > 0
            and len(self.running) < self.config.max_num_seqs
        ):
            seq = self.waiting[0]
            cached = self.cache.match_prefix(seq.token_ids)
            num_cached = (len(cached[0]) if cached else 0) * self.cache.block_size
            count = min(len(seq) - num_cached, budget)
            if not self.cache.try_allocate(seq.cache, num_cached + count, cached):
                break
            self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            seq.num_computed_tokens = num_cached
            seq.num_cached_tokens = num_cached
            self.num_cached_tokens += num_cached
            self.running.append(seq)
            batch.append(ScheduledSeq(seq, count))
            budget -= count
        return batch

    def postprocess(self, batch: list[ScheduledSeq], next_tokens: list[int | None]) -> list[Sequence]:
        """Advance the requests after a step.  ``next_tokens[i]`` is the token sampled for
        ``batch[i]``, or ``None`` when that entry was a portion that did not reach the end
        of its prompt.  The end-of-sequence token stays in the output."""
        finished: list[Sequence] = []
        for item, token in zip(batch, next_tokens, strict=True):
            seq = item.seq
            seq.num_computed_tokens += item.num_tokens
            self.cache.register_computed(seq.cache, seq.token_ids, seq.num_computed_tokens)
            self.cache.release_behind_window(seq.cache, seq.num_computed_tokens)
            if token is None:
                continue
            seq.token_ids.append(int(token))
            if self._is_done(seq, int(token)):
                seq.status = SequenceStatus.FINISHED
                self.cache.free(seq.cache)
                self.running.remove(seq)
                finished.append(seq)
        return finished

    def _is_done(self, seq: Sequence, token: int) -> bool:
        if not seq.params.ignore_eos and token in self.eos_token_ids:
            return True
        return seq.num_output_tokens >= seq.params.max_tokens

    def _preempt(self, seq: Sequence) -> None:
        self.running.remove(seq)
        self.cache.free(seq.cache)
        seq.status = SequenceStatus.WAITING
        seq.num_computed_tokens = 0
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)
