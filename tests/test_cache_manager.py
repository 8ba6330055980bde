"""The host side of the cache: no page lost, held twice or freed twice, under random orders."""

from __future__ import annotations

import random

import pytest

from tokamak_b200.cache.manager import (CacheManager, KVGroup, KVPagesNeed, OutOfPagesError,
                                        OutOfSlotsError, PageAllocator, StateGroup, StateNeed)


def manager(num_pages=8, page=4, window=None, slots=4, second_group=False):
    groups = [KVGroup(KVPagesNeed(2, 16, window), num_pages, page, ["l0", "l1"])]
    if second_group:
        groups.append(KVGroup(KVPagesNeed(2, 16, 6), num_pages, page, ["l2"]))
    return CacheManager(groups, [StateGroup(StateNeed((8,)), ["s0"])], slots)


def test_allocator_is_lifo_and_guards_double_free():
    a = PageAllocator(4)
    assert a.take(2) == [0, 1]
    a.give_back([0])
    assert a.take(1) == [0]                 # most recently freed first
    with pytest.raises(OutOfPagesError):
        a.take(3)
    assert a.num_free == 2                  # nothing changed
    a.give_back([1])
    with pytest.raises(AssertionError):
        a.give_back([1])


def test_grow_is_idempotent_append_only_and_all_or_nothing():
    m = manager(num_pages=4, page=4)
    m.admit("a")
    m.grow("a", 5)
    g = m.kv_groups[0]
    first = list(g.table("a"))
    assert len(first) == 2
    m.grow("a", 5); m.grow("a", 8)
    assert g.table("a") == first
    m.grow("a", 9)
    assert g.table("a")[:2] == first and len(g.table("a")) == 3
    m.admit("b")
    with pytest.raises(OutOfPagesError):
        m.grow("b", 8)                      # needs 2, one free
    assert g.table("b") == [] and g.num_free == 1
    assert not m.fits("b", 8) and m.fits("b", 4)
    m.check_invariants()


def test_free_is_idempotent_and_pages_come_back_lifo():
    m = manager()
    m.admit("a"); m.grow("a", 12)
    pages = list(m.kv_groups[0].table("a"))
    slot = m.slot("a")
    m.free("a"); m.free("a")
    assert m.kv_groups[0].num_free == 8 and m.num_free_slots == 4
    m.admit("b"); m.grow("b", 4)
    assert m.kv_groups[0].table("b") == [pages[-1]]     # the page freed last is used first
    assert m.slot("b") == slot
    m.check_invariants()


def test_slots_run_out_and_fresh_slots_are_flagged():
    m = manager(slots=2)
    m.admit("a"); m.admit("b")
    with pytest.raises(OutOfSlotsError):
        m.admit("c")
    with pytest.raises(ValueError):
        m.admit("a")
    assert m.fresh_slots == {m.slot("a"), m.slot("b")}
    m.free("a")
    m.admit("c")
    assert m.slot("c") in m.fresh_slots


def test_window_pages_are_given_back_as_the_window_passes():
    m = manager(num_pages=6, page=4, window=6)
    g = m.kv_groups[0]
    m.admit("a")
    m.grow("a", 8)
    m.advance("a", 8)                       # next query at 8 sees keys 3.. : page 0 still live
    assert g.released("a") == 0
    m.grow("a", 12); m.advance("a", 4)      # next query at 12 sees keys 7.. : page 0 is dead
    assert g.released("a") == 1 and g.num_free == 4
    stale = g.table("a")[0]
    m.admit("b"); m.grow("b", 4)
    assert g.table("b") == [stale]          # used again while "a" still lists it
    for n in range(13, 41):
        m.grow("a", n); m.advance("a", 1)
        m.check_invariants()
    assert len(g.held_pages("a")) <= 3      # bounded by the window, not by the length
    m.free("a"); m.free("b")
    assert g.num_free == 6
    assert g.peak_pages(1000, 1) <= 3 and g.peak_pages(1000, 16) <= 7


def test_groups_grow_together_or_not_at_all():
    m = manager(num_pages=3, page=4, second_group=True)
    m.admit("a"); m.grow("a", 12)
    m.admit("b")
    with pytest.raises(OutOfPagesError):
        m.grow("b", 4)
    assert all(g.table("b") == [] for g in m.kv_groups)
    m.advance("a", 12)                      # the windowed group gives pages back, the full one not
    assert m.kv_groups[1].num_free > 0 and m.kv_groups[0].num_free == 0
    assert not m.fits("b", 4)
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    m = manager(num_pages=12, page=4, slots=5, second_group=True)
    lengths: dict = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.num_free_slots:
            m.admit(next_id); lengths[next_id] = 0; next_id += 1
        elif op < 0.8 and lengths:
            rid = rng.choice(list(lengths))
            n = rng.choice([1, 1, 1, 2, 3, 7])
            try:
                m.grow(rid, lengths[rid] + n)
                m.advance(rid, n)
                lengths[rid] += n
            except OutOfPagesError:
                victim = rng.choice(list(lengths))
                m.free(victim); del lengths[victim]
        elif lengths:
            rid = rng.choice(list(lengths))
            m.free(rid); del lengths[rid]
            if rng.random() < 0.3:
                m.free(rid)
        m.check_invariants()
        for rid, n in lengths.items():
            assert m.length(rid) == n
            for g in m.kv_groups:
                assert len(g.table(rid)) >= g.pages_for(n)
    for rid in list(lengths):
        m.free(rid)
    assert all(g.num_free == g.num_pages for g in m.kv_groups) and m.num_free_slots == 5


def test_table_writes_follow_every_change_and_restart_keeps_the_slot():
    """The device learns of block tables write by write: new pages as (group, slot, index, page),
    entries of a request that ended or was restarted as -1.  A restart (preemption) gives the
    pages back, keeps the slot and marks the mixers' state in it for clearing."""
    from tokamak_b200.cache.manager import CacheManager, KVGroup, KVPagesNeed
    m = CacheManager([KVGroup(KVPagesNeed(1, 8), 6, 4, ["full"]),
                      KVGroup(KVPagesNeed(1, 8, window=5), 6, 4, ["win"])], [], 3)
    slot = m.admit("a")
    m.fresh_slots.clear()
    m.grow("a", 9)                                            # three pages in both groups
    assert sorted(m.table_writes) == sorted((g, slot, i, p) for g in (0, 1)
                                            for i, p in enumerate(m.kv_groups[g].table("a")))
    m.table_writes.clear()
    m.grow("a", 9)                                            # nothing new: nothing to write
    assert m.table_writes == []
    m.advance("a", 9)                                         # the window passed page 0 of group 1
    assert m.kv_groups[1].released("a") == 1 and m.table_writes == []    # the stale id stays, unread
    m.restart("a")
    assert m.has("a") and m.slot("a") == slot and m.length("a") == 0 and slot in m.fresh_slots
    assert sorted(m.table_writes) == [(g, slot, i, -1) for g in (0, 1) for i in range(3)]
    assert all(g.num_free == g.num_pages and g.table("a") == [] for g in m.kv_groups)
    m.check_invariants()
    m.table_writes.clear()
    m.grow("a", 4)
    m.free("a")
    assert m.table_writes[-2:] == [(0, slot, 0, -1), (1, slot, 0, -1)] and not m.has("a")
    assert m.num_free_slots == 3
    with pytest.raises(KeyError):
        m.restart("a")
    m.check_invariants()
