"""Device side of the cache: page pools, block tables and state records as tensors.

One pool tensor per group of key/value layers, laid out
``[cache key, k|v, page, kv head, slot in page, head_dim]`` so that the keys of
one (page, head) are one contiguous tile, and one ``[max_slots, max_pages]``
int32 block table per group, which mirrors the host manager's tables row by row.
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


class DeviceCache:
    """Tensors behind a :class:`CacheManager` and the copies that keep them in step with it."""

    def __init__(self, manager: CacheManager, dtype: torch.dtype, device: torch.device,
                 max_seq_len: int):
        self.manager = manager
        self.device = device
        self.dtype = dtype
        self._views: dict[Hashable, object] = {}
        self._pools: list[torch.Tensor] = []
        self._tables: list[torch.Tensor] = []
        self._host_tables: list[torch.Tensor] = []
        self._states: list[torch.Tensor] = []
        for g in manager.kv_groups:
            max_pages = -(-max_seq_len // g.page_size)
            pool = torch.zeros((len(g.cache_keys), 2, g.num_pages, g.need.n_kv_heads, g.page_size,
                                g.need.head_dim), dtype=dtype, device=device)
            table = torch.zeros((manager.max_slots, max_pages), dtype=torch.int32, device=device)
            host = torch.zeros((manager.max_slots, max_pages), dtype=torch.int32).pin_memory()
            self._pools.append(pool)
            self._tables.append(table)
            self._host_tables.append(host)
            for i, key in enumerate(g.cache_keys):
                self._views[key] = KVView(pool[i, 0], pool[i, 1], table, g.page_size, g.need.window)
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

    def sync(self) -> None:
        """Bring the device tables up to the host's and clear the records of fresh slots."""
        m = self.manager
        if m.dirty_rows:
            slot_req = {m.slot(r): r for r in m.live_requests()}
            for gi, slot in sorted(m.dirty_rows):
                req = slot_req.get(slot)
                if req is None:
                    continue
                pages = m.kv_groups[gi].table(req)
                host = self._host_tables[gi]
                if len(pages) > host.shape[1]:
                    raise RuntimeError(f"request {req!r} holds {len(pages)} pages, the table row "
                                       f"has room for {host.shape[1]}")
                host[slot, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
                self._tables[gi][slot].copy_(host[slot], non_blocking=True)
            m.dirty_rows.clear()
        if m.fresh_slots:
            for records in self._states:
                records[:, sorted(m.fresh_slots)] = 0
            m.fresh_slots.clear()

    def poison_free_pages(self, value: float = float("nan")) -> None:
        """Overwrite every page that no request holds (a test aid: stale reads then show)."""
        for g, pool in zip(self.manager.kv_groups, self._pools):
            free = list(g.allocator._free)
            if free:
                pool[:, :, torch.tensor(free, device=self.device)] = value
