"""Deciding what every step computes, and which step may be launched before its tokens are known.

The policy is the one of YuvGev00/mini-engine's scheduler (src/mini_engine/scheduler.py:44-159):
continuous batching under a token budget; requests that are running go first, in the order in
which they were admitted, each with as many of its outstanding tokens as the budget leaves (one
for a decoding request, a portion for a prompt); then waiting requests are admitted first come
first served, reusing cached prefix pages; when pages run out the most recently admitted request
is preempted and recomputed later.  This module states that policy for this engine:

* A step is planned as a :class:`StepPlan`: the scheduled items together with the
  :class:`~mini_engine_b200.engine.batch.StepEntry` list that the step function takes, so that
  nobody re-derives one from the other.
* The same place that plans a step also decides whether the decode step *after* it can be laid
  out and launched before this step's tokens have reached the host (:meth:`Scheduler.plan_ahead`),
  because that is a scheduling decision: it holds when the next plan is already certain (nobody
  can be admitted, everybody fits) and it takes the pages that the next plan would take.
* Pages are asked for through the cache manager, which grows the request's block table in every
  cache group or in none.

**When pages run out.**  The request that needs pages takes them from the tail of the running
list: the most recently admitted request gives back everything it holds (its pages in every
group, its state slot), keeps its tokens (generated ones included), has its computed count set
to zero and goes to the *front* of the waiting queue; this repeats until the pages are there or
the request that needs them is itself the one at the tail, in which case it is the one that
waits.  Requests at the tail have not been looked at yet when this happens, so a victim is never
part of the step being planned.  A step that preempted admits nobody.

Pure host code: no tensors.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from mini_engine_b200.cache.manager import CacheManager
from mini_engine_b200.engine.batch import StepEntry
from mini_engine_b200.engine.sequence import Sequence, SequenceStatus


@dataclass(frozen=True)
class SchedulerConfig:
    max_num_seqs: int = 16
    max_num_batched_tokens: int = 2048
    max_model_len: int = 4096


@dataclass
class ScheduledSeq:
    """``num_tokens`` tokens of ``seq`` from its ``num_computed_tokens`` on."""

    seq: Sequence
    num_tokens: int

    @property
    def samples(self) -> bool:
        """Whether this step reaches the end of the request, so that its logits are used."""
        return self.seq.num_computed_tokens + self.num_tokens == len(self.seq)

    def entry(self) -> StepEntry:
        """The same as the step function takes it: logits are wanted at the last token only, and
        only when the request's end is reached."""
        first = self.seq.num_computed_tokens
        want = (self.num_tokens - 1,) if self.samples else ()
        return StepEntry(self.seq.cache, first, self.seq.token_ids[first : first + self.num_tokens], want)


@dataclass
class StepPlan:
    """One step: what is scheduled and, in the same order, what the step function is given."""

    items: list[ScheduledSeq] = field(default_factory=list)
    entries: list[StepEntry] = field(default_factory=list)
    preempted: int = 0  # requests that lost their pages while this step was planned
    left_out: int = 0  # running requests that the token budget did not reach

    def grant(self, seq: Sequence, count: int) -> None:
        item = ScheduledSeq(seq, count)
        self.items.append(item)
        self.entries.append(item.entry())

    @property
    def decode_only(self) -> bool:
        return bool(self.items) and all(item.num_tokens == 1 and item.samples for item in self.items)


@dataclass
class AheadPlan:
    """The decode step after a planned one, as far as it can be known before that one's tokens
    are: its entries carry a placeholder token id each, and ``staying`` says which row of the
    planned step feeds which entry."""

    entries: list[StepEntry]
    staying: list[tuple[int, ScheduledSeq]]  # (row in the planned step, the item it came from)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager, eos_token_ids: set[int], rerun_safe: bool = True):
        """``rerun_safe``: whether a step that was launched ahead and then turns out not to be the
        next one may simply be dropped and planned anew.  That holds when a step leaves nothing
        behind but keys and values at the positions it computed (a rerun writes them again); it
        does not hold when a mixer advances a per-request state, so then no step is planned ahead."""
        self.config = config
        self.cache = cache
        self.eos_token_ids = set(eos_token_ids)
        self.rerun_safe = rerun_safe
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0
        self.num_cached_tokens = 0  # tokens served by the prefix cache, over all admissions

    # ------------------------------------------------------------------ submission

    def add(self, seq: Sequence) -> None:
        """Queue a request; one that could never run to its end is refused here, not later."""
        most = len(seq) + seq.params.max_tokens
        if most > self.config.max_model_len:
            raise ValueError(f"prompt + max_tokens = {most} exceeds max_model_len {self.config.max_model_len}")
        if self.cache.blocks_needed(most) > self.cache.smallest_pool:
            raise ValueError(f"request needs more than the {self.cache.smallest_pool} KV blocks available")
        seq.cache = self.cache.new_request()
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    # --------------------------------------------------------------------- a step

    def plan(self) -> StepPlan:
        plan = StepPlan()
        room = self.config.max_num_batched_tokens
        room = self._continue_running(plan, room)
        if plan.preempted == 0:
            self._admit_waiting(plan, room)
        return plan

    def schedule(self) -> list[ScheduledSeq]:
        """The items of the next step (the reference's name for :meth:`plan`)."""
        return self.plan().items

    def _continue_running(self, plan: StepPlan, room: int) -> int:
        """Every running request, oldest first, gets its next tokens while the budget lasts."""
        position = 0
        while position < len(self.running):
            seq = self.running[position]
            if room == 0:
                plan.left_out = len(self.running) - position
                break
            count = min(seq.num_uncomputed_tokens, room)
            if self._pages_for(seq, seq.num_computed_tokens + count, plan):
                plan.grant(seq, count)
                room -= count
                position += 1
            # else `seq` was the tail and is waiting now: position already names its successor (none)
        return room

    def _pages_for(self, seq: Sequence, num_tokens: int, plan: StepPlan) -> bool:
        """Pages for the first ``num_tokens`` tokens of a running request, taken from the requests
        admitted last if the pools are short.  False when ``seq`` itself had to give way."""
        while not self.cache.try_allocate(seq.cache, num_tokens):
            tail = self.running[-1]
            self._preempt(tail)
            plan.preempted += 1
            if tail is seq:
                return False
        return True

    def _admit_waiting(self, plan: StepPlan, room: int) -> None:
        """First come, first served: the head of the queue or nobody."""
        while self.waiting and room > 0 and len(self.running) < self.config.max_num_seqs:
            seq = self.waiting[0]
            shared = self.cache.match_prefix(seq.token_ids)
            reused = self.cache.block_size * (len(shared[0]) if shared else 0)
            count = min(len(seq) - reused, room)
            if not self.cache.try_allocate(seq.cache, reused + count, shared):
                return
            self.waiting.popleft()
            self.running.append(seq)
            seq.status = SequenceStatus.RUNNING
            seq.num_computed_tokens = seq.num_cached_tokens = reused
            self.num_cached_tokens += reused
            plan.grant(seq, count)
            room -= count

    # ------------------------------------------------------- the step after, ahead of time

    def plan_ahead(self, plan: StepPlan) -> AheadPlan | None:
        """The decode step that follows ``plan`` (itself a decode step that was just launched), if
        it is certain what it holds unless a request ends on an end-of-sequence token or a new
        request arrives in between: then the caller may launch it at once and check later
        (``Prepacked.matches``) that it was the right one.

        It is certain when (1) ``plan`` covers every running request, so the budget cuts nobody
        out; (2) nobody can be admitted: no request waits, or every place stays taken by requests
        that go on; (3) every request that goes on can have the pages of one more token without
        anybody being preempted.  Requests that reach their ``max_tokens`` with the token being
        drawn now are known to end and are left out.  The pages taken here are the ones the next
        :meth:`plan` would take; a request that ends instead gives all its pages back anyway."""
        if not self.rerun_safe or not plan.decode_only:
            return None
        if plan.left_out or len(plan.items) != len(self.running):
            return None
        going_on = [
            (row, item) for row, item in enumerate(plan.items)
            if item.seq.num_output_tokens + 1 < item.seq.params.max_tokens
        ]  # fmt: skip
        if not going_on:
            return None
        if self.waiting and len(going_on) < self.config.max_num_seqs:
            return None
        entries = []
        for _row, item in going_on:
            seq = item.seq
            first = seq.num_computed_tokens + 1  # the step in flight computes one token
            if first + 1 > self.config.max_model_len:
                return None
            if not self.cache.try_allocate(seq.cache, first + 1):
                return None  # pages already taken for earlier rows are the ones those rows need next anyway
            entries.append(StepEntry(seq.cache, first, [0], (0,)))
        return AheadPlan(entries, going_on)

    # --------------------------------------------------------------- after a step

    def postprocess(self, batch: list[ScheduledSeq], next_tokens: list[int | None]) -> list[Sequence]:
        """Book a step that ran.  ``next_tokens[i]`` is the token drawn for ``batch[i]``, or
        ``None`` for a portion that did not reach its request's end.  Computed pages are hashed
        for reuse, pages behind a window go back, a drawn token is appended (an end-of-sequence
        token stays in the output) and requests that are done give everything back."""
        done: list[Sequence] = []
        for item, token in zip(batch, next_tokens, strict=True):
            seq = item.seq
            seq.num_computed_tokens += item.num_tokens
            self.cache.register_computed(seq.cache, seq.token_ids, seq.num_computed_tokens)
            self.cache.release_behind_window(seq.cache, seq.num_computed_tokens)
            if token is None:
                continue
            token = int(token)
            seq.token_ids.append(token)
            if self._ends(seq, token):
                self._retire(seq)
                done.append(seq)
        return done

    def _ends(self, seq: Sequence, token: int) -> bool:
        if seq.num_output_tokens >= seq.params.max_tokens:
            return True
        return token in self.eos_token_ids and not seq.params.ignore_eos

    def _retire(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.FINISHED
        self.running.remove(seq)
        self.cache.free(seq.cache)

    def _preempt(self, seq: Sequence) -> None:
        """Recompute preemption: everything the request holds goes back, its tokens stay."""
        self.running.remove(seq)
        self.cache.free(seq.cache)
        seq.status = SequenceStatus.WAITING
        seq.num_computed_tokens = 0
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)
