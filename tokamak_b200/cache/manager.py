"""Host side of the cache: pages, block tables and per-request state slots.

Pure Python, no device: the scheduler asks it what fits, and the device side
(:mod:`tokamak_b200.cache.device`) mirrors its tables.

Layers whose cache needs are the same form a *group*.  A group of key/value
pages has a pool of pages of its own, one block table per live request, and a
rule for giving pages back: when the request ends, and, for a group whose layers
see only a window of keys, as soon as the window has passed a page.  Position
``p`` of a request lies in ``table[p // page_size]`` at offset ``p % page_size``
(the reference's mapping, src/tokamak/memory/block_manager.py:4-7).  The free
list is last-in first-out (block_manager.py:47-48), growth is all-or-nothing and
leaves the state intact when it fails (block_manager.py:74-93), and freeing is
idempotent (block_manager.py:131-140).

Beside the pages every live request owns one *slot*, an index below
``max_slots`` that addresses its row in the device block tables, its record in
every group of fixed-size state, and the engine's own record (position, sampling
parameters, generator counter, last token).  A request that is preempted gives
its pages back and keeps its slot (:meth:`CacheManager.restart`), as the reference
keeps a preempted request's generator (src/tokamak/engine/llm.py:339-340,441-445):
what can be recomputed from the tokens is dropped, what cannot stays.

Every change of a block table is also queued as a *table write* ``(group, slot,
logical index, page id)``, with ``-1`` for an entry whose page went back to the pool when
its request ended, so the device side applies the differences instead of copying rows.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable


class OutOfPagesError(RuntimeError):
    """A pool cannot provide the pages that were asked for."""


class OutOfSlotsError(RuntimeError):
    """Every request slot is taken."""


@dataclass(frozen=True)
class KVPagesNeed:
    """Cache need of a mixer that stores keys and values per position.

    ``window`` is the number of most recent positions a query sees (itself
    included), or ``None`` when it sees all of them.
    """

    n_kv_heads: int
    head_dim: int
    window: int | None = None
    kind: str = "kv_pages"


@dataclass(frozen=True)
class StateNeed:
    """Cache need of a mixer that keeps one record of fixed shape per request."""

    shape: tuple[int, ...]
    dtype: str = "float32"
    kind: str = "state"


class PageAllocator:
    """A fixed pool of page ids with a last-in first-out free list."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError(f"num_pages must be >= 1, got {num_pages}")
        self.num_pages = num_pages
        # page 0 is handed out first (src/tokamak/memory/block_manager.py:48)
        self._free = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, count: int) -> list[int]:
        if count > len(self._free):
            raise OutOfPagesError(f"{count} page(s) wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            if self._held[page]:
                raise AssertionError(f"page {page} handed out twice")
            self._held[page] = True
        return pages

    def give_back(self, pages: list[int]) -> None:
        for page in pages:
            if not self._held[page]:
                raise AssertionError(f"page {page} freed twice")
            self._held[page] = False
            self._free.append(page)


@dataclass
class _RequestPages:
    table: list[int] = field(default_factory=list)   # page id per logical page index, append-only
    released: int = 0                                # logical pages [0, released) were given back


class KVGroup:
    """Pages and block tables of one group of layers."""

    def __init__(self, need: KVPagesNeed, num_pages: int, page_size: int, cache_keys: list[Hashable]):
        if page_size < 1:
            raise ValueError(f"page_size must be >= 1, got {page_size}")
        self.need = need
        self.page_size = page_size
        self.cache_keys = list(cache_keys)
        self.allocator = PageAllocator(num_pages)
        self._requests: dict[Hashable, _RequestPages] = {}

    @property
    def num_pages(self) -> int:
        return self.allocator.num_pages

    @property
    def num_free(self) -> int:
        return self.allocator.num_free

    def pages_for(self, num_tokens: int) -> int:
        if num_tokens < 0:
            raise ValueError(f"num_tokens must be >= 0, got {num_tokens}")
        return -(-num_tokens // self.page_size)

    def first_live_page(self, next_position: int) -> int:
        """Logical index of the first page a query at ``next_position`` or later can see."""
        if self.need.window is None:
            return 0
        return max(0, next_position - self.need.window + 1) // self.page_size

    def shortfall(self, req_id: Hashable, num_tokens: int) -> int:
        """Pages to take from the pool so that ``num_tokens`` positions are covered."""
        held = len(self._requests[req_id].table) if req_id in self._requests else 0
        return max(0, self.pages_for(num_tokens) - held)

    def peak_pages(self, num_tokens: int, max_portion: int) -> int:
        """Most pages one request holds at a time when it grows to ``num_tokens``
        in portions of at most ``max_portion`` tokens."""
        if self.need.window is None:
            return self.pages_for(num_tokens)
        span = min(num_tokens, self.need.window - 1 + max(1, max_portion))
        return min(self.pages_for(num_tokens), self.pages_for(span) + 1)

    def table(self, req_id: Hashable) -> list[int]:
        entry = self._requests.get(req_id)
        return entry.table if entry else []

    def released(self, req_id: Hashable) -> int:
        entry = self._requests.get(req_id)
        return entry.released if entry else 0

    def grow(self, req_id: Hashable, num_tokens: int) -> list[tuple[int, int]]:
        """Cover ``num_tokens`` positions; returns the new (logical index, page id) pairs."""
        entry = self._requests.setdefault(req_id, _RequestPages())
        need = self.pages_for(num_tokens) - len(entry.table)
        if need <= 0:
            return []
        pages = self.allocator.take(need)   # raises before anything changed
        start = len(entry.table)
        entry.table.extend(pages)
        return [(start + i, page) for i, page in enumerate(pages)]

    def release_passed(self, req_id: Hashable, next_position: int) -> int:
        """Give back the pages that no query at ``next_position`` or later can see.

        The table keeps the stale ids (src/tokamak/memory/block_manager.py:95-129);
        attention never looks below the window, so they are never followed.
        """
        entry = self._requests.get(req_id)
        if entry is None:
            return 0
        upto = min(self.first_live_page(next_position), len(entry.table))
        if upto <= entry.released:
            return 0
        self.allocator.give_back(entry.table[entry.released:upto])
        count = upto - entry.released
        entry.released = upto
        return count

    def free(self, req_id: Hashable) -> None:
        entry = self._requests.pop(req_id, None)
        if entry is not None:
            self.allocator.give_back(entry.table[entry.released:])

    def held_pages(self, req_id: Hashable) -> list[int]:
        entry = self._requests.get(req_id)
        return entry.table[entry.released:] if entry else []


class StateGroup:
    """Fixed-size records, one per request slot, for every cache key of the group."""

    def __init__(self, need: StateNeed, cache_keys: list[Hashable]):
        self.need = need
        self.cache_keys = list(cache_keys)


class CacheManager:
    """All groups of a model, the request slots, and the bookkeeping between them."""

    def __init__(self, kv_groups: list[KVGroup], state_groups: list[StateGroup], max_slots: int):
        if max_slots < 1:
            raise ValueError(f"max_slots must be >= 1, got {max_slots}")
        self.kv_groups = kv_groups
        self.state_groups = state_groups
        self.max_slots = max_slots
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._slot_of: dict[Hashable, int] = {}
        self._length: dict[Hashable, int] = {}     # positions of each live request already in the cache
        # slots whose mixer state records must be cleared before their next use
        self.fresh_slots: set[int] = set()
        # block-table entries that the device has not seen yet: (group, slot, logical index, page id)
        self.table_writes: list[tuple[int, int, int, int]] = []

    # ---- slots ---------------------------------------------------------------------
    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def has(self, req_id: Hashable) -> bool:
        return req_id in self._slot_of

    def slot(self, req_id: Hashable) -> int:
        return self._slot_of[req_id]

    def live_requests(self) -> list[Hashable]:
        return list(self._slot_of)

    def admit(self, req_id: Hashable) -> int:
        """Give the request a slot; its state records start cleared."""
        if req_id in self._slot_of:
            raise ValueError(f"request {req_id!r} is already live")
        if not self._free_slots:
            raise OutOfSlotsError(f"all {self.max_slots} request slots are taken")
        slot = self._free_slots.pop()
        self._slot_of[req_id] = slot
        self._length[req_id] = 0
        self.fresh_slots.add(slot)
        return slot

    def length(self, req_id: Hashable) -> int:
        """Positions of the request that the cache holds (0 for an unknown request)."""
        return self._length.get(req_id, 0)

    def advance(self, req_id: Hashable, count: int) -> int:
        """Record that ``count`` more positions were written; gives back pages a window has passed."""
        self._length[req_id] += count
        self.release_passed(req_id, self._length[req_id])
        return self._length[req_id]

    # ---- pages ---------------------------------------------------------------------
    def fits(self, req_id: Hashable, num_tokens: int) -> bool:
        """Whether every group can cover ``num_tokens`` positions of the request now."""
        return all(g.shortfall(req_id, num_tokens) <= g.num_free for g in self.kv_groups)

    def grow(self, req_id: Hashable, num_tokens: int) -> None:
        """Cover ``num_tokens`` positions in every group, or change nothing and raise."""
        if req_id not in self._slot_of:
            raise KeyError(f"request {req_id!r} has no slot; admit it first")
        for g in self.kv_groups:
            short = g.shortfall(req_id, num_tokens)
            if short > g.num_free:
                raise OutOfPagesError(
                    f"request {req_id!r} needs {short} more page(s) for {num_tokens} tokens, "
                    f"but only {g.num_free} of {g.num_pages} are free")
        slot = self._slot_of[req_id]
        for gi, g in enumerate(self.kv_groups):
            for index, page in g.grow(req_id, num_tokens):
                self.table_writes.append((gi, slot, index, page))

    def release_passed(self, req_id: Hashable, next_position: int) -> int:
        """Give back, in every windowed group, the pages that the window has passed."""
        return sum(g.release_passed(req_id, next_position) for g in self.kv_groups)

    def _drop_pages(self, req_id: Hashable, slot: int) -> None:
        for gi, g in enumerate(self.kv_groups):
            # the row is void from now on: a stale id that a kernel followed would be a live
            # page of someone else, so the device's copy is overwritten with -1
            self.table_writes.extend((gi, slot, index, -1) for index in range(len(g.table(req_id))))
            g.free(req_id)

    def free(self, req_id: Hashable) -> None:
        """Give back the pages and the slot of a request; unknown ids are ignored."""
        slot = self._slot_of.pop(req_id, None)
        self._length.pop(req_id, None)
        if slot is not None:
            self._drop_pages(req_id, slot)
            self._free_slots.append(slot)
            self.fresh_slots.discard(slot)

    def restart(self, req_id: Hashable) -> None:
        """Preemption: the pages go back and the request starts over from position 0, in the
        slot it has.  State that mixers keep in the slot cannot be recomputed from pages and is
        cleared before the slot's next use; the engine's own record is left as it is."""
        slot = self._slot_of[req_id]
        self._drop_pages(req_id, slot)
        self._length[req_id] = 0
        self.fresh_slots.add(slot)

    def fits_empty_pool(self, num_tokens: int, max_portion: int) -> bool:
        """Whether one request of ``num_tokens`` tokens fits when it has the pools to itself."""
        return all(g.peak_pages(num_tokens, max_portion) <= g.num_pages for g in self.kv_groups)

    def check_invariants(self) -> None:
        """Every page is either free or held by exactly one request; slots likewise."""
        for g in self.kv_groups:
            held: list[int] = []
            for req_id in list(g._requests):
                held.extend(g.held_pages(req_id))
            free = list(g.allocator._free)
            if len(set(held)) != len(held):
                raise AssertionError("a page is held twice")
            if set(held) & set(free):
                raise AssertionError("a page is both held and free")
            if len(held) + len(free) != g.num_pages or len(set(free)) != len(free):
                raise AssertionError("a page was lost or is free twice")
        slots = list(self._slot_of.values())
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_slots:
            raise AssertionError("a slot was lost")
