"""Device side of the cache: page pools, block tables and state records as tensors.

One pool tensor per group of key/value layers, laid out
``[cache key, k|v, page, kv head, slot in page, head_dim]`` so that the keys of
one (page, head) are one contiguous tile, and one ``[max_slots, max_pages]``
int32 block table per group, which follows the host manager's tables write by write.
Pages are not cleared when they are given back
(src/tokamak/memory/paged_cache.py:51-52 clears only at start): a position is
always written before it is read.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable

import torch

from .manager import CacheManager, KVGroup, KVPagesNeed, StateGroup, StateNeed

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class KVView:
    """What a mixer sees of its cache: its key and value pages and its group's table."""

    k: torch.Tensor          # [num_pages, n_kv_heads, page_size, head_dim]
    v: torch.Tensor
    table: torch.Tensor      # [max_slots, max_pages] int32
    page_size: int
    window: int | None


@dataclass
class StateView:
    """Fixed-size records of one cache key: ``records[slot]`` belongs to the request in that slot."""

    records: torch.Tensor    # [max_slots, *shape]


def plan_groups(needs: dict[Hashable, object], pool_tokens: int, page_size: int
                ) -> tuple[list[KVGroup], list[StateGroup]]:
    """Group cache keys by need; every key/value group gets pages for ``pool_tokens`` tokens."""
    kv: dict[KVPagesNeed, list[Hashable]] = {}
    st: dict[StateNeed, list[Hashable]] = {}
    for key, need in needs.items():
        if isinstance(need, KVPagesNeed):
            kv.setdefault(need, []).append(key)
        elif isinstance(need, StateNeed):
            st.setdefault(need, []).append(key)
        else:
            raise TypeError(f"cache key {key!r} has an unknown kind of need: {need!r}")
    num_pages = -(-pool_tokens // page_size)
    return ([KVGroup(need, num_pages, page_size, keys) for need, keys in kv.items()],
            [StateGroup(need, keys) for need, keys in st.items()])


SLOT_WORDS = 8      # words of the engine's per-slot record; csrc/step_state.cu has the layout
REC_COMPUTED, REC_COUNTER, REC_SEED_LO, REC_SEED_HI, REC_TEMPERATURE, REC_TOP_K, REC_TOP_P, REC_LAST_TOKEN = range(8)


class DeviceCache:
    """Tensors behind a :class:`CacheManager`: page pools, block tables, mixer state records and
    the engine's own per-slot records.

    The block tables of all groups are one int32 tensor ``[group, slot, logical page]`` that starts
    at -1 everywhere; it changes only through the table writes that the manager queues, which the
    kernel that opens a step applies (:meth:`take_updates`).  The engine's records
    ``[slot, SLOT_WORDS]`` change the same way when a request is admitted, and on the device when
    a step advances a position or samples a token.
    """

    def __init__(self, manager: CacheManager, dtype: torch.dtype, device: torch.device,
                 max_seq_len: int):
        self.manager = manager
        self.device = device
        self.dtype = dtype
        self._views: dict[Hashable, object] = {}
        self._pools: list[torch.Tensor] = []
        self._states: list[torch.Tensor] = []
        page_sizes = {g.page_size for g in manager.kv_groups}
        if len(page_sizes) > 1:
            raise ValueError(f"all key/value groups share one page size, got {sorted(page_sizes)}")
        page_size = page_sizes.pop() if page_sizes else 1
        self.max_pages = -(-max_seq_len // page_size)
        self.tables = torch.full((max(1, len(manager.kv_groups)), manager.max_slots, self.max_pages), -1,
                                 dtype=torch.int32, device=device)
        self.slot_records = torch.zeros((manager.max_slots, SLOT_WORDS), dtype=torch.int32, device=device)
        self.slot_records[:, REC_LAST_TOKEN] = -1
        self._record_writes: dict[int, tuple[int, list[int]]] = {}
        for gi, g in enumerate(manager.kv_groups):
            pool = torch.zeros((len(g.cache_keys), 2, g.num_pages, g.need.n_kv_heads, g.page_size,
                                g.need.head_dim), dtype=dtype, device=device)
            self._pools.append(pool)
            for i, key in enumerate(g.cache_keys):
                self._views[key] = KVView(pool[i, 0], pool[i, 1], self.tables[gi], g.page_size, g.need.window)
        for g in manager.state_groups:
            records = torch.zeros((len(g.cache_keys), manager.max_slots, *g.need.shape),
                                  dtype=_STATE_DTYPES[g.need.dtype], device=device)
            self._states.append(records)
            for i, key in enumerate(g.cache_keys):
                self._views[key] = StateView(records[i])

    def view(self, cache_key: Hashable):
        return self._views[cache_key]

    def pools(self) -> list[torch.Tensor]:
        return self._pools

    def bytes_per_token(self) -> int:
        """Bytes of keys and values that one position occupies over all layers."""
        total = 0
        for g, pool in zip(self.manager.kv_groups, self._pools):
            total += len(g.cache_keys) * 2 * g.need.n_kv_heads * g.need.head_dim * pool.element_size()
        return total

    # ---- the engine's records ----------------------------------------------------------------
    def write_record(self, slot: int, *, temperature: float, top_k: int, top_p: float, seed: int,
                     counter: int = 0, fresh: bool = True) -> None:
        """Queue a slot's record for the next step's updates.  ``fresh`` (a newly admitted request)
        also puts the position to 0 and the last token to none; without it only the sampling
        parameters, the seed and the counter are replaced."""
        import struct
        if not 0 <= slot < min(self.manager.max_slots, 1 << 16):
            raise ValueError(f"slot {slot} is outside the records")
        bits = lambda x: struct.unpack("<i", struct.pack("<f", float(x)))[0]
        wrap = lambda x: ((int(x) & 0xFFFFFFFF) ^ 0x80000000) - 0x80000000      # as a signed word
        seed &= 0x7FFFFFFFFFFFFFFF
        words = [0, int(counter), wrap(seed), wrap(seed >> 32), bits(temperature), int(top_k),
                 bits(top_p), -1]
        mask = 0xFF if fresh else 0x7E
        old = self._record_writes.get(slot)
        if old is not None and not fresh:
            # an earlier write for the slot is still queued: keep the words this one leaves alone
            mask |= old[0]
            words[0], words[7] = old[1][0], old[1][7]
        self._record_writes[slot] = (mask, words)

    @property
    def updates_pending(self) -> bool:
        return bool(self._record_writes or self.manager.table_writes)

    def take_updates(self) -> tuple[list[int], list[int]]:
        """What the device has not seen yet, as the two payloads of the update list: record writes
        ``(slot, 8 words)`` and table writes ``(flat index, page id)``, the last write of an
        entry only (the kernel applies them in no particular order)."""
        rec: list[int] = []
        for slot, (mask, words) in self._record_writes.items():
            rec.append(slot | (mask << 16))
            rec.extend(words)
        self._record_writes.clear()
        m = self.manager
        last: dict[int, int] = {}
        per_group = m.max_slots * self.max_pages
        for gi, slot, index, page in m.table_writes:
            if index >= self.max_pages:
                raise RuntimeError(f"slot {slot} holds page index {index}, the table row has room "
                                   f"for {self.max_pages}")
            last[gi * per_group + slot * self.max_pages + index] = page
        m.table_writes.clear()
        tab = [x for at, page in last.items() for x in (at, page)]
        return rec, tab

    def clear_fresh_state(self) -> None:
        """Zero the mixer state records of slots that were handed out or restarted."""
        m = self.manager
        if m.fresh_slots:
            if self._states:
                index = torch.tensor(sorted(m.fresh_slots), dtype=torch.long, device=self.device)
                for records in self._states:
                    records.index_fill_(1, index, 0)
            m.fresh_slots.clear()

    def read_record(self, slot: int) -> dict:
        """The engine's record of a slot as the device holds it now (synchronises; for tests and tools)."""
        import struct
        w = self.slot_records[slot].tolist()
        flt = lambda x: struct.unpack("<f", struct.pack("<i", x))[0]
        return {"num_computed": w[REC_COMPUTED], "counter": w[REC_COUNTER],
                "seed": (w[REC_SEED_LO] & 0xFFFFFFFF) | ((w[REC_SEED_HI] & 0xFFFFFFFF) << 32),
                "temperature": flt(w[REC_TEMPERATURE]), "top_k": w[REC_TOP_K], "top_p": flt(w[REC_TOP_P]),
                "last_token": w[REC_LAST_TOKEN]}

    def poison_free_pages(self, value: float = float("nan")) -> None:
        """Overwrite every page that no request holds (a test aid: stale reads then show)."""
        for g, pool in zip(self.manager.kv_groups, self._pools):
            free = list(g.allocator._free)
            if free:
                pool[:, :, torch.tensor(free, device=self.device)] = value
