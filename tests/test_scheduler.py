"""Scheduler decisions, driven by hand without a model (after the reference's
tests/unit/test_scheduler.py): sequences are advanced exactly as the engine would."""

from __future__ import annotations

import pytest

from tokamak_b200.cache.manager import CacheManager, KVGroup, KVPagesNeed, OutOfPagesError
from tokamak_b200.engine.scheduler import Scheduler
from tokamak_b200.engine.sequence import FinishReason, Sequence, SequenceStatus
from tokamak_b200.sampling import SamplingParams


def make(num_pages=8, page=4, slots=4, batch=4, budget=64, chunk=None):
    m = CacheManager([KVGroup(KVPagesNeed(1, 16), num_pages, page, ["l0"])], [], slots)
    return m, Scheduler(m, batch, budget, chunk)


def seq(i, n_prompt, max_new=8):
    return Sequence(i, list(range(1, n_prompt + 1)), SamplingParams(temperature=0.0, max_new_tokens=max_new))


def run_plan(manager, plan, token=9, finish_at=None):
    """What the engine does after a step: advance the cache, append sampled tokens, free finished."""
    for e in plan.entries:
        manager.advance(e.seq.seq_id, e.count)
        e.seq.num_computed = e.start + e.count
    for e in plan.entries:
        if e.samples:
            done = e.seq.append_checked(token, eos_token_ids=(), max_total_tokens=10 ** 6)
            if done:
                manager.free(e.seq.seq_id)


def describe(plan):
    return [(e.seq.seq_id, e.start, e.count, e.samples) for e in plan.entries]


def test_fcfs_admission_under_a_token_budget_and_chunk():
    m, s = make(num_pages=32, budget=16, chunk=8)
    a, b, c = seq(0, 20), seq(1, 5), seq(2, 3)
    for x in (a, b, c):
        s.add(x)
    p = s.schedule()
    assert describe(p) == [(0, 0, 8, False), (1, 0, 5, True), (2, 0, 3, True)]   # 16 tokens, in order
    run_plan(m, p)
    p = s.schedule()
    # decodes first (one token each), then the running prefill's next portion
    assert describe(p) == [(1, 5, 1, True), (2, 3, 1, True), (0, 8, 8, False)]
    run_plan(m, p)
    p = s.schedule()
    assert describe(p) == [(1, 6, 1, True), (2, 4, 1, True), (0, 16, 4, True)]
    run_plan(m, p)
    assert a.num_output_tokens == 1 and b.num_output_tokens == 3


def test_budget_smaller_than_the_decodes_serves_the_oldest():
    m, s = make(num_pages=32, budget=2)
    for i in range(3):
        s.add(seq(i, 1))
    run_plan(m, s.schedule())            # admits 0 and 1 (one token each)
    p = s.schedule()
    assert describe(p) == [(0, 1, 1, True), (1, 1, 1, True)]       # 2 waits: no budget left


def test_batch_size_gate_and_finish_frees_pages():
    m, s = make(batch=2)
    a, b, c = seq(0, 4, max_new=1), seq(1, 4), seq(2, 4)
    for x in (a, b, c):
        s.add(x)
    p = s.schedule()
    assert [e.seq.seq_id for e in p.entries] == [0, 1]
    run_plan(m, p)
    assert a.is_finished and a.finish_reason is FinishReason.LENGTH
    p = s.schedule()
    assert [e.seq.seq_id for e in p.entries] == [1, 2]              # 2 takes the place of 0
    assert m.kv_groups[0].table(0) == []


def test_page_gate_makes_the_head_wait_and_nobody_overtakes():
    m, s = make(num_pages=4, page=4)
    a, b, c = seq(0, 12), seq(1, 8), seq(2, 2)
    for x in (a, b, c):
        s.add(x)
    p = s.schedule()
    assert [e.seq.seq_id for e in p.entries] == [0]                 # 1 does not fit; 2 must not overtake
    run_plan(m, p)
    assert [e.seq.seq_id for e in s.schedule().entries] == [0]


def test_preemption_evicts_the_newest_and_requeues_at_the_front():
    m, s = make(num_pages=4, page=4, budget=64)
    a, b = seq(0, 7), seq(1, 7)
    s.add(a); s.add(b)
    run_plan(m, s.schedule())            # both prefilled: 2 pages each, pool full
    waiting_late = seq(2, 2)
    s.add(waiting_late)
    p = s.schedule()                     # a and b decode token 8: fits in their last page
    assert [e.seq.seq_id for e in p.entries] == [0, 1] and not p.preempted
    run_plan(m, p)
    p = s.schedule()                     # token 9 of a needs a third page: b is evicted
    assert p.preempted == [b]
    assert [e.seq.seq_id for e in p.entries] == [0]
    assert b.status is SequenceStatus.WAITING and b.num_computed == 0 and b.num_output_tokens == 2
    assert list(s.waiting) == [b, waiting_late]                     # ahead of what arrived later
    # the pages are back, the slot (with the record of its random generator) is kept
    assert m.kv_groups[0].table(1) == [] and m.has(1) and m.length(1) == 0
    slot_of_b = m.slot(1)
    assert p.admitted == []
    run_plan(m, p)
    while not a.is_finished:
        run_plan(m, s.schedule())
    p = s.schedule()                     # b resumes over prompt + generated, then samples the next
    assert describe(p)[0] == (1, 0, 9, True)
    assert b.num_preemptions == 1 and s.num_preemptions == 1
    assert m.slot(1) == slot_of_b and b not in p.admitted           # resumed, not admitted anew


def test_a_starving_sequence_may_evict_itself():
    m, s = make(num_pages=2, page=4)
    a = seq(0, 8, max_new=4)
    s.add(a)
    run_plan(m, s.schedule())
    with pytest.raises(OutOfPagesError, match="pool can ever provide"):
        s.schedule()                     # 9 tokens never fit 2 pages: evicts itself, then cannot re-admit


def test_none_when_done_and_validation():
    m, s = make()
    assert s.schedule() is None and not s.has_unfinished()
    a = seq(0, 3, max_new=1)
    s.add(a)
    assert s.has_unfinished()
    run_plan(m, s.schedule())
    assert s.schedule() is None
    with pytest.raises(ValueError):
        Scheduler(m, 0, 8)
    with pytest.raises(ValueError):
        Scheduler(m, 2, 0)
    with pytest.raises(ValueError):
        Scheduler(m, 99, 8)


def test_stop_rules_in_the_reference_order():
    a = Sequence(0, [1, 2], SamplingParams(max_new_tokens=3))
    assert not a.append_checked(5, eos_token_ids=(7,), max_total_tokens=100)
    assert a.append_checked(7, eos_token_ids=(7,), max_total_tokens=100)
    assert a.finish_reason is FinishReason.STOP and a.output_token_ids == [5, 7]
    b = Sequence(1, [1, 2], SamplingParams(max_new_tokens=3, ignore_eos=True))
    b.append_checked(7, eos_token_ids=(7,), max_total_tokens=100)
    b.append_checked(7, eos_token_ids=(7,), max_total_tokens=100)
    assert b.append_checked(7, eos_token_ids=(7,), max_total_tokens=100)
    assert b.finish_reason is FinishReason.LENGTH
    c = Sequence(2, [1, 2, 3], SamplingParams(max_new_tokens=50))
    assert c.append_checked(4, eos_token_ids=(), max_total_tokens=4)
    assert c.finish_reason is FinishReason.LENGTH
    assert c.tokens_from(2, 2) == [3, 4] and c.tokens_from(0, 4) == [1, 2, 3, 4]
    with pytest.raises(RuntimeError):
        c.append_output_token(1)
    with pytest.raises(ValueError):
        Sequence(3, [], SamplingParams())


def launch(m, plan):
    """What the engine does when it launches a planned step: lengths and cursors move on."""
    for e in plan.entries:
        m.advance(e.seq.seq_id, e.count)
        e.seq.num_computed = e.start + e.count


def arrive(plan, token=9, limit=10 ** 6):
    """The tokens of a launched step are read."""
    for e in plan.entries:
        if e.samples and not e.seq.is_finished:
            e.seq.append_checked(token, eos_token_ids=(), max_total_tokens=limit)


def test_plan_ahead_while_a_step_is_in_flight():
    """The step after a launched step is planned before its tokens are known: every sequence it
    samples for brings one more token that only the device has, prompt portions go on, waiting
    requests are admitted into free room, and sequences that reach their length limit in the step
    in flight are left out."""
    m, s = make(num_pages=16, page=4, budget=64)
    a, b = seq(0, 5, max_new=3), seq(1, 6, max_new=8)
    s.add(a); s.add(b)
    limit = lambda q: 10 ** 6
    first = s.schedule()                                # both prompts whole
    launch(m, first)
    dec = s.plan_ahead(first, limit)
    assert describe(dec) == [(0, 5, 1, True), (1, 6, 1, True)]     # their first tokens are still on the device
    assert a.num_tokens == 5 and a.num_tokens_due == 6
    arrive(first)
    launch(m, dec)
    ahead = s.plan_ahead(dec, limit)
    assert describe(ahead) == [(0, 6, 1, True), (1, 7, 1, True)]
    assert m.length(0) == 6 and m.length(1) == 7        # lengths advance at launch, not at planning
    arrive(dec)
    launch(m, ahead)
    # sequence 0 has two of its three tokens: the step in flight gives the third, so it drops out
    nxt = s.plan_ahead(ahead, limit)
    assert describe(nxt) == [(1, 8, 1, True)]
    assert a.ending and not b.ending
    arrive(ahead)
    assert a.is_finished
    launch(m, nxt)
    # a context limit does the same
    assert s.plan_ahead(nxt, lambda q: q.num_tokens + 1) is None
    # somebody waiting is admitted beside the token in flight (sequence 0 still holds its pages)
    c = seq(2, 3)
    s.add(c)
    with_c = s.plan_ahead(nxt, limit)
    assert describe(with_c) == [(1, 9, 1, True), (2, 0, 3, True)] and with_c.admitted == [c]
    m.check_invariants()


def test_plan_ahead_carries_prompt_portions_on():
    m, s = make(num_pages=64, page=4, slots=4, batch=4, budget=16, chunk=8)
    a, b = seq(0, 3, max_new=8), seq(1, 20, max_new=8)
    s.add(a)
    first = s.schedule()
    launch(m, first)
    s.add(b)
    plan = s.plan_ahead(first, lambda q: 10 ** 6)
    assert describe(plan) == [(0, 3, 1, True), (1, 0, 8, False)]
    arrive(first)
    launch(m, plan)
    plan2 = s.plan_ahead(plan, lambda q: 10 ** 6)
    assert describe(plan2) == [(0, 4, 1, True), (1, 8, 8, False)]
    arrive(plan)
    launch(m, plan2)
    plan3 = s.plan_ahead(plan2, lambda q: 10 ** 6)
    assert describe(plan3) == [(0, 5, 1, True), (1, 16, 4, True)]
    arrive(plan2)
    launch(m, plan3)
    plan4 = s.plan_ahead(plan3, lambda q: 10 ** 6)
    assert describe(plan4) == [(0, 6, 1, True), (1, 20, 1, True)]
    m.check_invariants()


def test_plan_ahead_gives_up_when_pages_are_short():
    m2, s2 = make(num_pages=2, page=4, budget=64)
    c = seq(1, 7, max_new=8)
    s2.add(c)
    run_plan(m2, s2.schedule())                         # 7 computed, token 8 sampled
    dec = s2.schedule()                                 # position 7: still inside page 2
    assert describe(dec) == [(1, 7, 1, True)]
    launch(m2, dec)
    assert s2.plan_ahead(dec, lambda q: 10 ** 6) is None    # position 8 would need a third page
    m2.check_invariants()


def test_watermark_keeps_room_for_the_running_and_never_blocks_a_lone_request():
    # 16 pages of 4 positions; a quarter of them (4 pages) stays free while anything runs
    m = CacheManager([KVGroup(KVPagesNeed(1, 16), 16, 4, ["l0"])], [], 4)
    s = Scheduler(m, 4, 256, None, watermark=0.25)
    a, b, c = seq(0, 24), seq(1, 24), seq(2, 8)         # 6 + 6 + 2 pages
    for x in (a, b, c):
        s.add(x)
    p = s.schedule()
    # a is alone when it is admitted (no margin asked); b would leave 4 free: just allowed;
    # c would leave 2: it waits although its pages are free, and nobody overtakes
    assert [e.seq.seq_id for e in p.entries] == [0, 1]
    run_plan(m, p)
    assert [e.seq.seq_id for e in s.schedule().entries] == [0, 1]
    assert m.kv_groups[0].num_free >= 2 and c.status is SequenceStatus.WAITING
    # without the margin all three start at once
    m2 = CacheManager([KVGroup(KVPagesNeed(1, 16), 16, 4, ["l0"])], [], 4)
    s2 = Scheduler(m2, 4, 256, None)
    for x in (seq(0, 24), seq(1, 24), seq(2, 8)):
        s2.add(x)
    assert [e.seq.seq_id for e in s2.schedule().entries] == [0, 1, 2]
    # a request that is alone is admitted whenever it fits, whatever the margin
    m3 = CacheManager([KVGroup(KVPagesNeed(1, 16), 16, 4, ["l0"])], [], 4)
    s3 = Scheduler(m3, 4, 256, None, watermark=0.9)
    s3.add(seq(0, 60))
    assert [e.seq.seq_id for e in s3.schedule().entries] == [0]
    with pytest.raises(ValueError):
        Scheduler(m3, 4, 256, None, watermark=1.0)


@pytest.mark.parametrize("seed", range(12))
def test_random_workloads_finish_in_arrival_order_with_every_page_accounted_for(seed):
    """Random requests through small pools (a full and a windowed group), with random budgets,
    portion sizes and margins: every step keeps the cache's invariants, plans only what the pages
    cover, never lets a later arrival start before an earlier one has, and every request ends with
    exactly its tokens, preempted or not."""
    import random
    rng = random.Random(seed)
    page = rng.choice((2, 4, 8))
    window = rng.choice((None, 3 * page, 5 * page + 1))
    n_pages = rng.randint(12, 40)
    groups = [KVGroup(KVPagesNeed(1, 16), n_pages, page, ["full"])]
    if window is not None:
        groups.append(KVGroup(KVPagesNeed(1, 16, window=window), n_pages, page, ["windowed"]))
    slots = rng.randint(2, 6)
    m = CacheManager(groups, [], slots)
    budget = rng.randint(max(slots, 4), 48)
    chunk = rng.choice((None, 2, 5, 16))
    s = Scheduler(m, slots, budget, chunk, watermark=rng.choice((0.0, 0.0, 0.2)))
    most = (n_pages - 1) * page                        # every request fits the empty pool alone
    seqs = []
    for i in range(rng.randint(5, 14)):
        n_prompt = rng.randint(1, max(1, most // 2))
        max_new = rng.randint(1, max(1, min(20, most - n_prompt)))
        q = seq(i, n_prompt, max_new)
        seqs.append(q)
        s.add(q)
    started: list[int] = []
    given_slots: set[int] = set()
    steps = 0
    while s.has_unfinished():
        plan = s.schedule()
        assert plan is not None and plan.entries
        steps += 1
        assert steps < 20000, "the scheduler makes no progress"
        assert plan.num_tokens <= budget
        ids = [e.seq.seq_id for e in plan.entries]
        assert len(set(ids)) == len(ids) and len(s.running) <= slots
        for e in plan.entries:
            assert e.seq.status is SequenceStatus.RUNNING and e.count >= 1
            assert e.start == e.seq.num_computed == m.length(e.seq.seq_id)
            assert chunk is None or e.count <= chunk or e.count == 1
            assert e.samples == (e.start + e.count == e.seq.num_tokens)
            for g in m.kv_groups:                      # the pages of the planned positions are there
                assert len(g.table(e.seq.seq_id)) >= g.pages_for(e.start + e.count)
            if e.start == 0 and e.seq.seq_id not in started:
                started.append(e.seq.seq_id)
        for v in plan.preempted:
            assert v.status is SequenceStatus.WAITING and v.num_computed == 0
            assert m.has(v.seq_id) and m.length(v.seq_id) == 0
            assert all(g.table(v.seq_id) == [] for g in m.kv_groups)
        for q in plan.admitted:                        # a slot for the first time: exactly once each
            assert q.seq_id not in given_slots
            given_slots.add(q.seq_id)
        assert all(e.seq.seq_id in given_slots for e in plan.entries)
        run_plan(m, plan, token=rng.randrange(1, 50))
        m.check_invariants()
    assert started == sorted(started)                  # first starts happen in arrival order
    for q in seqs:
        assert q.is_finished and q.num_output_tokens == q.sampling_params.max_new_tokens
    assert not m.live_requests()
    assert all(g.num_free == g.num_pages for g in m.kv_groups)


def test_a_step_is_cut_down_to_a_multiple_of_the_token_tile():
    """536 tokens would be five tiles of 128 in every matrix product; the portion gives 24 up."""
    m = CacheManager([KVGroup(KVPagesNeed(1, 16), 400, 16, ["l0"])], [], 64)
    s = Scheduler(m, 64, 544, 512, token_multiple=128)
    for i in range(24):
        s.add(seq(i, 3, max_new=50))
    plan = s.schedule()
    assert plan.num_tokens == 72                       # fewer than a tile: left as it is
    run_plan(m, plan)
    long = seq(99, 2000, max_new=5)
    s.add(long)
    plan = s.schedule()
    assert plan.num_tokens == 512 and [e.count for e in plan.entries if e.seq is long] == [488]
    run_plan(m, plan)
    plan = s.schedule()
    assert plan.num_tokens == 512
    entry = [e for e in plan.entries if e.seq is long][0]
    assert (entry.start, entry.count, entry.samples) == (488, 488, False)    # nothing lost, nothing twice


def test_a_portion_that_ends_its_prompt_is_not_cut():
    m, s = make(num_pages=100, page=16, budget=2048)
    s = Scheduler(m, 4, 2048, None, token_multiple=128)
    s.add(seq(0, 300))
    plan = s.schedule()
    assert [(e.count, e.samples) for e in plan.entries] == [(300, True)]
