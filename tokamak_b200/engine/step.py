"""The step function: one batch of (request, its next tokens) through the model.

The reference runs either one whole prompt or one token of every running
sequence per step (src/tokamak/engine/llm.py:347-388).  Here a step is a flat
batch of tokens: portions of prompts beside single decoded tokens, cut anywhere.
Every entry continues its request at the position the cache has reached, the
step writes the new keys and values first and then attends over everything up
to each token (the reference's order, src/tokamak/model/step_context.py:88), and
logits are produced only for the places that are asked for.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from ..cache.device import DeviceCache
from ..csrc import ops

_ERR_NAMES = {1: "token id outside the vocabulary", 2: "page outside the pool or the table",
              3: "negative position", 4: "request row outside the batch",
              5: "a bounded wait in a kernel ran out"}


class StepError(RuntimeError):
    """A kernel reported bad input through the error word."""


def _bucket(length: int) -> int:
    bucket = 256
    while bucket < length:
        bucket *= 2
    return bucket


@dataclass
class StepEntry:
    """Next tokens of one request and the places among them whose logits are wanted.

    ``tokens=None`` stands for one token: the one that the request sampled last, which is still
    on the device (in the request's slot record) and may not have been read by the host yet."""

    req_id: Hashable
    tokens: Sequence[int] | None
    want: Sequence[int] = ()

    @property
    def count(self) -> int:
        return 1 if self.tokens is None else len(self.tokens)


@dataclass
class SamplingRow:
    """How a request samples (see tokamak_b200.sampling); ``counter`` is the index of its next draw."""

    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    counter: int = 0


@dataclass
class StepBatch:
    """Device-side description of a step, handed to every part.

    All index tensors are int32.  ``tok_req[t]`` is the row of token ``t``'s
    request in the per-request arrays; ``req_slot[r]`` is that request's row in the
    block tables and state records; ``req_kv_len[r]`` counts the positions of the
    request after this step, so its tokens sit at ``req_kv_len - req_q_len ...``.
    The ``host_*`` lists repeat the per-request numbers for parts that plan on the host;
    a part that reads them must not declare itself ``GRAPH_SAFE`` (``parts/base.py``).
    """

    n_tokens: int
    n_reqs: int
    n_want: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    tok_req: torch.Tensor
    req_q_start: torch.Tensor
    req_q_len: torch.Tensor
    req_kv_len: torch.Tensor
    req_slot: torch.Tensor
    logits_rows: torch.Tensor
    decode_items: torch.Tensor      # token indices of requests that bring one token
    prefill_items: torch.Tensor     # token indices of requests that bring more than one
    prefill_tiles: torch.Tensor     # [n_tiles, 2] (request row, 64-token tile) of those requests, longest first
    prefill_tc: "ops.PrefillItems"  # the same requests as the work list of the tcgen05 kernel
    cache: DeviceCache
    err: torch.Tensor
    host_q_start: list[int] = field(default_factory=list)
    host_q_len: list[int] = field(default_factory=list)
    host_kv_len: list[int] = field(default_factory=list)
    host_slot: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0     # a bound on the longest context: the next power of two, at least 256, so
                            # that what kernels plan from it (grids, key splits) changes rarely
    scratch: dict = field(default_factory=dict)     # per-step values that parts share (e.g. plans)
    row_slot: torch.Tensor | None = None            # slot of the request of every wanted row


@dataclass
class PendingStep:
    """A launched step whose sampled tokens have not been read yet (see ``StepFunction.collect``)."""

    n_want: int
    host: torch.Tensor          # pinned: error word, then the sampled tokens
    done: torch.cuda.Event


class _PinnedRing:
    """A few pinned host buffers used in turn as the source of asynchronous copies: a buffer is
    written again only after the copy that read it has completed."""

    def __init__(self, words: int, ring: int = 3):
        self.hosts = [torch.zeros(max(1, words), dtype=torch.int32).pin_memory() for _ in range(ring)]
        self.events: list = [None] * ring
        self.turn = 0

    def next(self) -> tuple[torch.Tensor, int]:
        i = self.turn
        self.turn = (i + 1) % len(self.hosts)
        if self.events[i] is not None:
            self.events[i].synchronize()
        return self.hosts[i], i

    def copied(self, i: int) -> None:
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()


class StepBuffers:
    """Everything at a fixed device address that describes steps, and the pinned staging behind it.

    * ``dev``: the integers of a step that the host lays out (token ids, positions, the
      per-request arrays, ...), one copy per such step.
    * ``updates``: the list of record and table writes that the kernel opening the next step
      applies; copied only when something changed.
    * ``dec_*``: the description of a step of single next tokens, which the device derives from
      the slot records; only the list of slots comes from the host, and only when it changed.
    * ``result``: error word and sampled tokens, which travel back together.
    """

    RING = 3

    def __init__(self, cache: DeviceCache, max_tokens: int):
        device, max_reqs = cache.device, cache.manager.max_slots
        self.device = device
        sms = ops.sm_count(device) if device.type == "cuda" else 148
        # the prefill work list: a record per 256 tokens of a request, and up to 2 sms more for parts
        self.capacity = (10 * max_reqs + 12 * max_tokens + 64
                         + ops.PREFILL_TC_RECORD * (max_tokens // ops.PREFILL_TC_ROWS + max_reqs + 2 * sms + 8))
        self.sms = sms
        self.staging = _PinnedRing(self.capacity, self.RING)
        self.dev = torch.zeros(self.capacity, dtype=torch.int32, device=device)
        max_tab = cache.tables.numel()
        self.ctl_words = 2 + 9 * max_reqs + 2 * max_tab
        self.ctl_ring = _PinnedRing(self.ctl_words, self.RING)
        ctl = torch.zeros(self.ctl_words, dtype=torch.int32, device=device)
        self.updates = ops.UpdateBuffers(ctl, max_reqs, max_tab, cache.slot_records, cache.tables)
        self.dec_ring = _PinnedRing(max_reqs, self.RING)
        self.dec_slots = torch.zeros(max_reqs, dtype=torch.int32, device=device)
        self.dec_slots_host: list[int] | None = None       # what the device holds in dec_slots
        self.dec_token_ids = torch.zeros(max_reqs, dtype=torch.int32, device=device)
        self.dec_positions = torch.zeros(max_reqs, dtype=torch.int32, device=device)
        self.dec_kv_len = torch.zeros(max_reqs, dtype=torch.int32, device=device)
        self.iota = torch.arange(max_reqs, dtype=torch.int32, device=device)
        self.ones = torch.ones(max_reqs, dtype=torch.int32, device=device)
        self.empty = torch.zeros(0, dtype=torch.int32, device=device)
        self.result = torch.zeros(4 + max_tokens, dtype=torch.int32, device=device)
        self.result_hosts = [torch.zeros(4 + max_tokens, dtype=torch.int32).pin_memory()
                             for _ in range(self.RING)]
        self.result_turn = 0
        self.h2d_bytes = 0          # bytes copied to the device so far, counted from the copies made
        self.h2d_copies = 0
        self.d2h_bytes = 0

    def _copy(self, dst: torch.Tensor, ring: _PinnedRing, host: torch.Tensor, i: int, words: int) -> None:
        dst[:words].copy_(host[:words], non_blocking=True)
        ring.copied(i)
        self.h2d_bytes += 4 * words
        self.h2d_copies += 1

    def upload(self, arrays: list[np.ndarray]) -> list[torch.Tensor]:
        """Copy the arrays (int32 views) to the device in one transfer; returns device views."""
        total = sum(a.size for a in arrays)
        if total > self.capacity:
            raise ValueError(f"step needs {total} staging words, capacity is {self.capacity}")
        host, i = self.staging.next()
        host_np = host.numpy()
        views = []
        off = 0
        for a in arrays:
            host_np[off:off + a.size] = a
            views.append(self.dev[off:off + a.size])
            off += a.size
        if total:
            self._copy(self.dev, self.staging, host, i, total)
        return views

    def upload_updates(self, rec: list[int], tab: list[int]) -> None:
        """Send the update list (record writes, table writes) for the next opening kernel."""
        n_rec, n_tab = len(rec) // 9, len(tab) // 2
        if n_rec > self.updates.max_rec or n_tab > self.updates.max_tab:
            raise ValueError(f"{n_rec} record and {n_tab} table writes exceed the update list")
        host, i = self.ctl_ring.next()
        words = 2 + len(rec) + len(tab)
        host_np = host.numpy()
        host_np[0], host_np[1] = n_rec, n_tab
        host_np[2:2 + len(rec)] = rec
        host_np[2 + len(rec):words] = tab
        self._copy(self.updates.ctl, self.ctl_ring, host, i, words)

    def upload_dec_slots(self, slots: list[int]) -> None:
        if slots == self.dec_slots_host:
            return
        host, i = self.dec_ring.next()
        host.numpy()[:len(slots)] = slots
        self._copy(self.dec_slots, self.dec_ring, host, i, len(slots))
        self.dec_slots_host = list(slots)


class StepFunction:
    """Builds the batch description, runs the model and keeps the cache's lengths.

    Two kinds of step.  A *laid-out* step is described by the host: any mix of prompt portions
    and single tokens; its description is uploaded and ``step_begin`` opens it.  A *state-driven*
    step is one in which every request brings the token it sampled last and wants the next one
    sampled: the device derives tokens, positions and lengths from the slot records
    (``decode_begin``), the host uploads only what changed (the list of slots, new pages), and
    because its launches are the same every time it is replayed from a CUDA graph where every
    part of the model allows that (``GRAPH_SAFE``, see ``parts/base.py``).
    """

    def __init__(self, model, cache: DeviceCache, max_step_tokens: int, max_seq_len: int,
                 use_graphs: bool = True):
        self.model = model
        self.use_graphs = use_graphs
        self._graphs: dict = {}          # (batch, key-length bucket) -> captured decode step
        self._graph_seen: dict = {}
        self._graph_pool = None
        self.cache = cache
        self.manager = cache.manager
        self.device = cache.device
        self.max_step_tokens = max_step_tokens
        self.max_seq_len = max_seq_len
        self.buffers = StepBuffers(cache, max_step_tokens)
        self.graph_safe = bool(model is not None and getattr(model, "graph_safe", lambda: False)())
        # how many work items a part makes of one block of prompt tokens (its query heads, for an
        # attention mixer): the work list of prompt portions is balanced for the smallest
        parts = model.parts() if model is not None and hasattr(model, "parts") else []
        self.prefill_heads = min((p.prefill_heads for p in parts if getattr(p, "prefill_heads", None)), default=32)
        self.steps_run = 0
        self.graph_launches = 0      # kernels replayed from CUDA graphs (not counted by ops.LAUNCHES)
        self.graph_replays = 0

    # ---- request lifetime ------------------------------------------------------------
    def admit(self, req_id: Hashable, sampling: SamplingRow | None = None) -> None:
        """Give the request a slot and start its record (greedy unless ``sampling`` says otherwise)."""
        self.manager.admit(req_id)
        self.set_record(req_id, sampling or SamplingRow(), fresh=True)

    def set_record(self, req_id: Hashable, sampling: SamplingRow, fresh: bool = False) -> None:
        """Queue the request's record for the device: how it samples, its seed and the index of its
        next draw; ``fresh`` also starts position and last token anew (a newly admitted request)."""
        self.cache.write_record(self.manager.slot(req_id), temperature=sampling.temperature,
                                top_k=sampling.top_k, top_p=sampling.top_p, seed=sampling.seed,
                                counter=sampling.counter, fresh=fresh)

    def free(self, req_id: Hashable) -> None:
        self.manager.free(req_id)

    def restart(self, req_id: Hashable) -> None:
        """Preemption: pages back, position 0, slot and record kept."""
        self.manager.restart(req_id)

    def length(self, req_id: Hashable) -> int:
        return self.manager.length(req_id)

    def record(self, req_id: Hashable) -> dict:
        """The request's slot record as the device holds it (synchronises)."""
        return self.cache.read_record(self.manager.slot(req_id))

    # ---- the step ----------------------------------------------------------------------
    def _reserve(self, entries: Sequence[StepEntry]) -> tuple[list[int], list[int], list[int]]:
        """Slots, pages and the per-request numbers (tokens brought, start, slot) of a step."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        counts, starts, slots = [], [], []
        for e in entries:
            if e.req_id in seen:
                raise ValueError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if not self.manager.has(e.req_id):
                if e.tokens is None:
                    raise ValueError(f"request {e.req_id!r} is not live: it has no sampled token to go on from")
                self.admit(e.req_id)
            n = e.count
            if n < 1:
                raise ValueError(f"request {e.req_id!r} brings no tokens")
            start = self.manager.length(e.req_id)
            if start + n > self.max_seq_len:
                raise ValueError(f"request {e.req_id!r} would reach {start + n} tokens, "
                                 f"beyond max_seq_len={self.max_seq_len}")
            self.manager.grow(e.req_id, start + n)
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.req_id!r} wants place {w} of {n} tokens")
            counts.append(n)
            starts.append(start)
            slots.append(self.manager.slot(e.req_id))
        if sum(counts) > self.max_step_tokens:
            raise ValueError(f"step of {sum(counts)} tokens exceeds max_step_tokens={self.max_step_tokens}")
        return counts, starts, slots

    def _send_updates(self) -> None:
        self.cache.clear_fresh_state()
        if self.cache.updates_pending:
            self.buffers.upload_updates(*self.cache.take_updates())

    def build(self, entries: Sequence[StepEntry]) -> StepBatch:
        """Reserve pages, lay the batch out, upload its description and open the step on the device."""
        q_len, starts, slots = self._reserve(entries)
        n_reqs = len(entries)
        q_start = [0] * n_reqs
        n_tokens = 0
        for r in range(n_reqs):
            q_start[r] = n_tokens
            n_tokens += q_len[r]
        kv_len = [s + n for s, n in zip(starts, q_len)]
        tok_parts, pos_parts, req_parts, pf_parts = [], [], [], []
        rows, row_slot, dec_items, fed = [], [], [], []
        for r, e in enumerate(entries):
            n = q_len[r]
            rows.extend(q_start[r] + w for w in e.want)
            row_slot.extend(slots[r] for _ in e.want)
            tok_parts.append(np.zeros(1, dtype=np.int32) if e.tokens is None
                             else np.asarray(e.tokens, dtype=np.int32))
            fed.append(1 if e.tokens is None else 0)
            pos_parts.append(np.arange(starts[r], starts[r] + n, dtype=np.int32))
            req_parts.append(np.full(n, r, dtype=np.int32))
            if n == 1:
                dec_items.append(q_start[r])
            else:
                pf_parts.append(np.arange(q_start[r], q_start[r] + n, dtype=np.int32))

        i32 = lambda x: np.asarray(x, dtype=np.int32)
        cat = lambda parts: np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)

        def tiles_of(rows_per_tile: int) -> list[int]:
            # (request row, tile index) of every request that brings more than one token; tiles
            # with the most keys to visit start first
            tiles = [(kv_len[r] - q_len[r] + rows_per_tile * (t + 1), r, t) for r in range(n_reqs)
                     if q_len[r] > 1 for t in range(-(-q_len[r] // rows_per_tile))]
            tiles.sort(reverse=True)
            return [x for _, r, t in tiles for x in (r, t)]

        records, n_parts, n_split = ops.prefill_tc_records(q_start, q_len, kv_len, slots,
                                                            heads=self.prefill_heads, sms=self.buffers.sms)
        arrays = [cat(tok_parts), cat(pos_parts), cat(req_parts), i32(q_start), i32(q_len), i32(kv_len),
                  i32(slots), i32(rows), i32(dec_items), cat(pf_parts), i32(tiles_of(64)),
                  records.reshape(-1), i32(fed), i32(row_slot)]
        views = self.buffers.upload(arrays)
        self._send_updates()
        batch = StepBatch(
            n_tokens=n_tokens, n_reqs=n_reqs, n_want=len(rows),
            token_ids=views[0], positions=views[1], tok_req=views[2], req_q_start=views[3],
            req_q_len=views[4], req_kv_len=views[5], req_slot=views[6], logits_rows=views[7],
            decode_items=views[8], prefill_items=views[9], prefill_tiles=views[10],
            prefill_tc=ops.PrefillItems(views[11].view(-1, ops.PREFILL_TC_RECORD), n_parts, n_split),
            cache=self.cache, err=self.buffers.result[:4],
            host_q_start=q_start, host_q_len=q_len, host_kv_len=kv_len, host_slot=slots,
            max_q_len=max(q_len), max_kv_len=_bucket(max(kv_len)), row_slot=views[13])
        ops.step_begin(self.buffers.updates, batch.token_ids, batch.req_q_start, batch.req_kv_len,
                       batch.req_slot, views[12] if any(fed) else None, batch.err)
        return batch

    def _build_from_state(self, entries: Sequence[StepEntry]) -> StepBatch:
        """The description of a state-driven step: tensors at fixed addresses that ``decode_begin``
        fills on the device.  Uploads the list of slots if it differs from the device's, and the
        pending updates if there are any."""
        _, starts, slots = self._reserve(entries)
        b, n = self.buffers, len(entries)
        b.upload_dec_slots(slots)
        self._send_updates()
        return StepBatch(
            n_tokens=n, n_reqs=n, n_want=n,
            token_ids=b.dec_token_ids[:n], positions=b.dec_positions[:n], tok_req=b.iota[:n],
            req_q_start=b.iota[:n], req_q_len=b.ones[:n], req_kv_len=b.dec_kv_len[:n],
            req_slot=b.dec_slots[:n], logits_rows=b.iota[:n], decode_items=b.iota[:n],
            prefill_items=b.empty, prefill_tiles=b.empty,
            prefill_tc=ops.PrefillItems(b.empty.view(0, ops.PREFILL_TC_RECORD), 0, 0),
            cache=self.cache, err=b.result[:4],
            host_q_start=list(range(n)), host_q_len=[1] * n, host_kv_len=[s + 1 for s in starts],
            host_slot=slots, max_q_len=1, max_kv_len=_bucket(max(starts) + 1), row_slot=b.dec_slots[:n])

    def finish(self, entries: Sequence[StepEntry]) -> None:
        """Advance the lengths and give back the pages that a window has passed."""
        for e in entries:
            self.manager.advance(e.req_id, e.count)
        self.steps_run += 1

    @torch.inference_mode()
    def run(self, entries: Sequence[StepEntry], check: bool = True) -> torch.Tensor:
        """Float32 logits ``[wanted, vocab]`` on the device, in the order of entries and ``want``."""
        batch = self.build(entries)
        logits = self.model.forward(batch)
        self.finish(entries)
        if check:
            self.check_errors()
        return logits

    def run_and_sample(self, entries: Sequence[StepEntry],
                       sampling: Sequence[SamplingRow] | None = None) -> list[int]:
        """One token per wanted place, sampled on the device; one copy back for tokens and errors."""
        return self.collect(self.launch_and_sample(entries, sampling))

    @torch.inference_mode()
    def launch_and_sample(self, entries: Sequence[StepEntry],
                          sampling: Sequence[SamplingRow] | None = None) -> PendingStep:
        """Start a step that samples one token at every wanted place (at most one per entry) with
        the parameters, seed and counter of the request's slot record; ``collect`` reads them.

        ``sampling`` is a shorthand for callers that keep the parameters themselves: one row per
        wanted place, written into those requests' records before the step (their counters
        included).  The engine instead writes a record once, when a request is admitted.

        The step may be launched before the step before it has been collected: an entry with
        ``tokens=None`` takes the token it sampled there from its record, so the device never
        waits for the host between two steps.  At most two launched steps may be waiting to be
        collected, and they are collected in the order of their launch.
        """
        if any(len(e.want) > 1 for e in entries):
            raise ValueError("a sampling step takes at most one wanted place per request")
        if sampling is not None:
            wanting = [e for e in entries if e.want]
            if len(sampling) != len(wanting):
                raise ValueError(f"{len(sampling)} sampling rows for {len(wanting)} wanted places")
            for e, row in zip(wanting, sampling):
                if not self.manager.has(e.req_id):
                    self.admit(e.req_id, row)
                else:
                    self.set_record(e.req_id, row)
        res = self.buffers.result
        if all(e.tokens is None and len(e.want) == 1 for e in entries):
            batch = self._build_from_state(entries)
            self._run_from_state(batch)
        else:
            batch = self.build(entries)
            logits = self.model.forward(batch)
            if batch.n_want:
                ops.sample_slots(logits, self.cache.slot_records, batch.row_slot, res[4:4 + batch.n_want],
                                 batch.err)
        W = batch.n_want
        self.finish(entries)
        bufs = self.buffers
        host = bufs.result_hosts[bufs.result_turn]
        bufs.result_turn = (bufs.result_turn + 1) % bufs.RING
        host[:4 + W].copy_(res[:4 + W], non_blocking=True)
        bufs.d2h_bytes += 4 * (4 + W)
        done = torch.cuda.Event()
        done.record()
        return PendingStep(W, host, done)

    def _from_state_launches(self, batch: StepBatch) -> torch.Tensor:
        b, n = self.buffers, batch.n_reqs
        ops.decode_begin(b.updates, b.dec_slots, n, self.max_seq_len, b.dec_token_ids, b.dec_positions,
                         b.dec_kv_len, batch.err)
        logits = self.model.forward(batch)
        ops.sample_slots(logits, self.cache.slot_records, batch.row_slot, b.result[4:4 + n], batch.err)
        return logits

    def _run_from_state(self, batch: StepBatch) -> None:
        """A state-driven step: replayed from its CUDA graph where the model allows it (captured
        the second time a shape, batch size and bucket of the longest context, is seen), else
        launched kernel by kernel."""
        if self.use_graphs and self.graph_safe:
            key = (batch.n_tokens, batch.max_kv_len)     # kernels size their grids from the bucket
            graph = self._graphs.get(key)
            if graph is None and self._graph_seen.get(key, 0) >= 1:
                graph = self._capture(key, batch)
            if graph is not None:
                graph["graph"].replay()
                self.graph_launches += graph["kernels"]
                self.graph_replays += 1
                return
            self._graph_seen[key] = self._graph_seen.get(key, 0) + 1
        self._from_state_launches(batch)

    def collect(self, pending: PendingStep) -> list[int]:
        """Wait for a launched step and return its sampled tokens; raises on a kernel error."""
        pending.done.synchronize()
        self._raise_on_error(pending.host[:4].tolist())
        return pending.host[4:4 + pending.n_want].tolist()

    def _capture(self, key, batch: StepBatch) -> dict:
        """Record the state-driven step of this shape; its launches are replayed, not run, here."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self._from_state_launches(batch)
        kernels = ops.LAUNCHES - before
        ops.LAUNCHES = before
        entry = {"graph": graph, "kernels": kernels, "logits": logits}
        self._graphs[key] = entry
        return entry

    def check_errors(self) -> None:
        self._raise_on_error(self.buffers.result[:4].cpu().tolist())

    def _raise_on_error(self, word: list[int]) -> None:
        if word[0] != 0:
            self.buffers.result[:4].zero_()
            ops.reset_workspaces()      # counters that a kernel which gave up may have left non-zero
            raise StepError(f"kernel error {word[0]} ({_ERR_NAMES.get(word[0], 'unknown')}); "
                            f"details {word[1:]}")
