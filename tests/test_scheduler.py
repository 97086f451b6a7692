"""The scheduler's decisions, driven by a fake model that needs no tensors
(the method of tests/test_scheduler.py:19-22 of YuvGev00/mini-engine)."""

from __future__ import annotations

import random

import pytest

from mini_engine_b200.cache import CacheManager, GroupSpec
from mini_engine_b200.engine.scheduler import Scheduler, SchedulerConfig
from mini_engine_b200.engine.sequence import Sequence, SequenceStatus
from mini_engine_b200.sampling import SamplingParams

EOS = 99


def make(num_blocks=16, block_size=4, max_num_seqs=4, budget=64, max_model_len=64, prefix=True, groups=None):
    cache = CacheManager(groups or [GroupSpec("full")], num_blocks, block_size, max_num_seqs, prefix)
    return Scheduler(SchedulerConfig(max_num_seqs, budget, max_model_len), cache, {EOS}), cache


class Ran:
    """What one scheduled item was when it was scheduled (`samples` changes afterwards)."""

    def __init__(self, item):
        self.seq, self.num_tokens, self.samples = item.seq, item.num_tokens, item.samples


def step(sched, token=0):
    batch = sched.schedule()
    ran = [Ran(item) for item in batch]
    next_tokens = [token if item.samples else None for item in batch]
    return ran, sched.postprocess(batch, next_tokens)


def run_to_end(sched, token=0, limit=1000):
    steps = 0
    while sched.has_unfinished():
        batch, _ = step(sched, token)
        assert batch, "an empty batch while work is pending"
        steps += 1
        assert steps < limit
    return steps


def request(n, max_tokens=4, base=0, **kw):
    return Sequence([base + i for i in range(n)], SamplingParams(max_tokens=max_tokens, **kw))


def test_decodes_and_a_new_prompt_share_one_batch():
    sched, _ = make()
    first = request(5)
    sched.add(first)
    step(sched)
    sched.add(request(7, base=100))
    batch, _ = step(sched)
    assert [(i.seq is first, i.num_tokens) for i in batch] == [(True, 1), (False, 7)]


def test_run_to_completion_frees_everything():
    sched, cache = make()
    seqs = [request(n, base=100 * n) for n in (3, 9, 14)]
    for s in seqs:
        sched.add(s)
    run_to_end(sched)
    assert all(s.is_finished and s.num_output_tokens == 4 for s in seqs)
    assert cache.num_free_blocks == 16
    cache.check_invariants([])


def test_eos_and_ignore_eos():
    sched, _ = make()
    stops, ignores = request(3, max_tokens=5), request(3, max_tokens=5, base=50, ignore_eos=True)
    sched.add(stops), sched.add(ignores)
    run_to_end(sched, token=EOS)
    assert stops.output_token_ids == [EOS] and ignores.output_token_ids == [EOS] * 5


def test_request_cap():
    sched, _ = make(max_num_seqs=2)
    for i in range(3):
        sched.add(request(2, base=10 * i))
    batch, _ = step(sched)
    assert len(batch) == 2 and len(sched.waiting) == 1


def test_token_budget_cuts_prompts_and_nobody_jumps_the_queue():
    sched, _ = make(budget=8, prefix=False)
    long, short = request(13), request(2, base=100)
    sched.add(long), sched.add(short)
    batch, _ = step(sched)
    assert [(i.seq is long, i.num_tokens, i.samples) for i in batch] == [(True, 8, False)]
    batch, _ = step(sched)
    assert [(i.seq is long, i.num_tokens, i.samples) for i in batch] == [(True, 5, True), (False, 2, True)]
    assert long.num_output_tokens == 1 and short.num_output_tokens == 1


def test_admission_stops_at_the_first_request_that_does_not_fit():
    sched, _ = make(num_blocks=4, prefix=False)
    big, small = request(14, max_tokens=2), request(2, max_tokens=2, base=100)
    blocker = request(6, max_tokens=2, base=200)
    sched.add(blocker)
    step(sched)
    sched.add(big), sched.add(small)
    batch, _ = step(sched)
    assert [i.seq for i in batch] == [blocker]  # big needs 4 pages, 2 are free; small must wait behind it


def test_pages_run_out_newest_is_preempted_and_readmitted_first():
    sched, cache = make(num_blocks=4, block_size=4, prefix=False)
    old, new = request(7, max_tokens=8), request(7, max_tokens=8, base=100)
    sched.add(old), sched.add(new)
    step(sched)  # both prompts: 2 pages each, pool full
    step(sched)  # the 8th token of each still fits its second page
    batch, _ = step(sched)  # both need a third page: old gets it by preempting new
    assert [i.seq for i in batch] == [old]
    assert new.status is SequenceStatus.WAITING and new.num_computed_tokens == 0 and new.num_preemptions == 1
    assert sched.waiting[0] is new and sched.num_preemptions == 1
    assert new.num_output_tokens == 2  # the generated tokens are kept
    assert new.cache.holds_nothing()
    cache.check_invariants([old.cache])
    run_to_end(sched)
    assert old.num_output_tokens == 8 and new.num_output_tokens == 8
    cache.check_invariants([])


def test_a_request_that_is_its_own_victim_waits():
    sched, cache = make(num_blocks=2, block_size=4, prefix=False, max_model_len=8)
    only = request(4, max_tokens=4)
    sched.add(only)
    run_to_end(sched)
    assert only.num_output_tokens == 4 and cache.num_free_blocks == 2


def test_preempted_request_hits_its_own_prefix_on_return():
    sched, _ = make(num_blocks=6, block_size=4)
    first, second = request(8, max_tokens=12), request(8, max_tokens=12, base=100)
    sched.add(first), sched.add(second)
    run_to_end(sched)
    assert sched.num_preemptions > 0
    assert second.num_preemptions > 0 and second.num_cached_tokens > 0
    assert first.num_output_tokens == 12 and second.num_output_tokens == 12


def test_prefix_hit_skips_cached_tokens():
    sched, _ = make()
    a = request(9)
    sched.add(a)
    run_to_end(sched)
    b = request(9)  # the same prompt again
    sched.add(b)
    batch = sched.schedule()
    assert batch[0].num_tokens == 1 and b.num_computed_tokens == 8 and sched.num_cached_tokens == 8
    sched.postprocess(batch, [0])


def test_never_fitting_requests_are_rejected():
    sched, _ = make(num_blocks=4, block_size=4, max_model_len=32)
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add(request(30, max_tokens=4))
    with pytest.raises(ValueError, match="KV blocks"):
        sched.add(request(14, max_tokens=4))
    with pytest.raises(ValueError):
        Sequence([], SamplingParams())


def test_window_group_and_state_slots_under_the_scheduler():
    groups = [GroupSpec("full"), GroupSpec("win", window=6)]
    sched, cache = make(num_blocks=10, groups=groups)
    seqs = [request(n, max_tokens=10, base=100 * n) for n in (11, 5, 8)]
    for s in seqs:
        sched.add(s)
    while sched.has_unfinished():
        step(sched)
        cache.check_invariants([s.cache for s in sched.running])
        slots = [s.cache.state_slot for s in sched.running]
        assert len(set(slots)) == len(slots) and all(x >= 0 for x in slots)
    assert all(pool.num_free == 10 for pool in cache.pools)
    assert cache.slots.held == set()


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_with_every_invariant_kept(seed):
    rng = random.Random(seed)
    sched, cache = make(num_blocks=12, block_size=4, max_num_seqs=3, budget=rng.choice([5, 9, 64]), max_model_len=40)
    seqs = []
    for step_number in range(300):
        if rng.random() < 0.3 and len(seqs) < 25:
            shared = [1, 2, 3, 4, 5, 6, 7, 8] if rng.random() < 0.5 else []
            seq = Sequence(shared + [rng.randrange(10, 60) for _ in range(rng.randrange(1, 16))],
                           SamplingParams(max_tokens=rng.randrange(1, 12)))
            sched.add(seq)
            seqs.append(seq)
        if sched.has_unfinished():
            batch, _ = step(sched, token=rng.randrange(60))
            assert batch
            assert sum(i.num_tokens for i in batch) <= sched.config.max_num_batched_tokens
            assert len(sched.running) <= 3
        cache.check_invariants([s.cache for s in sched.running])
    run_to_end(sched)
    assert all(s.is_finished and s.num_output_tokens == s.params.max_tokens for s in seqs)
    cache.check_invariants([])


# ---------------------------------------------------------------- plans and the step after


def test_a_plan_carries_the_entries_of_its_items():
    sched, _ = make(budget=8, prefix=False)
    long, short = request(13), request(2, base=100)
    sched.add(long), sched.add(short)
    plan = sched.plan()
    assert [(e.start, list(e.token_ids), tuple(e.want)) for e in plan.entries] == [(0, list(range(8)), ())]
    assert plan.entries[0].cache is long.cache and not plan.decode_only
    sched.postprocess(plan.items, [None])
    plan = sched.plan()
    assert [(e.start, len(e.token_ids), tuple(e.want)) for e in plan.entries] == [(8, 5, (4,)), (0, 2, (1,))]
    sched.postprocess(plan.items, [7, 7])
    plan = sched.plan()  # both decode now
    assert plan.decode_only and [(e.start, list(e.token_ids), tuple(e.want)) for e in plan.entries] == [(13, [7], (0,)), (2, [7], (0,))]


def decoding(sched, seqs):
    """Adds the requests and runs steps until every one of them decodes."""
    for s in seqs:
        sched.add(s)
    while any(s.num_computed_tokens < s.num_prompt_tokens for s in seqs):
        step(sched)


def test_the_step_after_is_planned_when_it_is_certain():
    sched, cache = make(num_blocks=16, block_size=4)
    a, b = request(3, max_tokens=6), request(6, max_tokens=6, base=50)
    decoding(sched, [a, b])
    plan = sched.plan()
    free_before = cache.num_free_blocks
    ahead = sched.plan_ahead(plan)
    assert ahead is not None and [row for row, _ in ahead.staying] == [0, 1]
    # one position further than the step being run, a placeholder token each, logits wanted
    assert [(e.start, list(e.token_ids), tuple(e.want)) for e in ahead.entries] == [
        (a.num_computed_tokens + 1, [0], (0,)), (b.num_computed_tokens + 1, [0], (0,))]  # fmt: skip
    # `a` holds 4 tokens after this step and its next token opens a second page, taken here already
    assert len(a.cache.block_tables[0]) == 2 and cache.num_free_blocks == free_before - 1
    sched.postprocess(plan.items, [1, 1])
    following = sched.plan()
    assert [(e.cache, e.start) for e in following.entries] == [(e.cache, e.start) for e in ahead.entries]
    assert cache.num_free_blocks == free_before - 1  # the plan found its pages taken
    cache.check_invariants([a.cache, b.cache])


def test_requests_that_end_at_their_own_limit_are_left_out_of_the_step_after():
    sched, _ = make()
    ends, goes_on = request(3, max_tokens=2), request(5, max_tokens=9, base=50)
    decoding(sched, [ends, goes_on])  # each has one generated token now
    plan = sched.plan()
    ahead = sched.plan_ahead(plan)
    assert ahead is not None and [(row, item.seq) for row, item in ahead.staying] == [(1, goes_on)]
    assert len(ahead.entries) == 1 and ahead.entries[0].cache is goes_on.cache
    finished = sched.postprocess(plan.items, [1, 1])
    assert finished == [ends]
    assert [e.cache for e in sched.plan().entries] == [goes_on.cache]


def test_no_step_is_planned_ahead_when_the_next_plan_is_open():
    # a request waits and a place is free: the next step admits it
    sched, _ = make(max_num_seqs=2)
    first = request(3, max_tokens=8)
    decoding(sched, [first])
    plan = sched.plan()
    sched.waiting.append(Sequence([1, 2, 3], SamplingParams(max_tokens=2)))  # arrives while the step runs
    sched.waiting[-1].cache = sched.cache.new_request()
    assert sched.plan_ahead(plan) is None
    # ... unless every place stays taken
    sched, _ = make(max_num_seqs=2)
    pair = [request(3, max_tokens=8), request(4, max_tokens=8, base=30)]
    decoding(sched, pair)
    sched.add(request(2, max_tokens=2, base=60))
    plan = sched.plan()
    assert len(plan.items) == 2 and sched.plan_ahead(plan) is not None
    # a step with a prompt portion in it is no decode step
    sched, _ = make(budget=4)
    sched.add(request(9))
    assert sched.plan_ahead(sched.plan()) is None
    # pages for one more token cannot be had without preempting
    sched, cache = make(num_blocks=3, block_size=4, prefix=False, max_model_len=16)
    two = [request(3, max_tokens=5), request(3, max_tokens=5, base=40)]
    decoding(sched, two)  # 4 tokens each after the step planned now: a page each is full, one page is free
    plan = sched.plan()
    assert sched.plan_ahead(plan) is None
    cache.check_invariants([s.cache for s in sched.running])
    # the model's length limit ends a request with the token being drawn
    sched, _ = make(max_model_len=8)
    last = request(5, max_tokens=3)
    decoding(sched, [last])
    step(sched)
    plan = sched.plan()  # computes token 7 of 8: nothing can follow
    assert sched.plan_ahead(plan) is None


def test_no_step_is_planned_ahead_for_a_model_whose_steps_cannot_be_rerun():
    cache = CacheManager([GroupSpec("full")], 16, 4, 4, True)
    sched = Scheduler(SchedulerConfig(4, 64, 64), cache, {EOS}, rerun_safe=False)
    one = request(3, max_tokens=8)
    decoding(sched, [one])
    plan = sched.plan()
    assert plan.decode_only and sched.plan_ahead(plan) is None
