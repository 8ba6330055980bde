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


@dataclass
class StepEntry:
    """Next tokens of one request and the places among them whose logits are wanted."""

    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class SamplingRow:
    """How to sample at one wanted place (see tokamak_b200.sampling)."""

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
    The ``host_*`` lists repeat the per-request numbers for parts that plan on the host.
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
    prefill_tiles_tc: torch.Tensor  # the same in the tile size of the tcgen05 kernel (ops.PREFILL_TC_ROWS)
    cache: DeviceCache
    err: torch.Tensor
    host_q_start: list[int] = field(default_factory=list)
    host_q_len: list[int] = field(default_factory=list)
    host_kv_len: list[int] = field(default_factory=list)
    host_slot: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    scratch: dict = field(default_factory=dict)     # per-step values that parts share (e.g. plans)


@dataclass
class PendingStep:
    """A launched step whose sampled tokens have not been read yet (see ``StepFunction.collect``)."""

    n_want: int
    host: torch.Tensor          # pinned: error word, then the sampled tokens
    done: torch.cuda.Event


class StepBuffers:
    """Pinned host staging and its device twin for the integers that describe a step.

    The host side is a small ring: a copy to the device is asynchronous, so a staging
    buffer is written again only after the copy that read it has completed.
    """

    RING = 3

    def __init__(self, device: torch.device, max_tokens: int, max_reqs: int):
        self.device = device
        self.capacity = 8 * max_reqs + 12 * max_tokens + 64
        self.hosts = [torch.zeros(self.capacity, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events: list = [None] * self.RING
        self.turn = 0
        self.dev = torch.zeros(self.capacity, dtype=torch.int32, device=device)
        # error word and sampled tokens travel back together
        self.result = torch.zeros(4 + max_tokens, dtype=torch.int32, device=device)
        self.result_hosts = [torch.zeros(4 + max_tokens, dtype=torch.int32).pin_memory()
                             for _ in range(self.RING)]
        self.result_turn = 0

    def upload(self, arrays: list[np.ndarray]) -> list[torch.Tensor]:
        """Copy the arrays (int32 views) to the device in one transfer; returns device views."""
        total = sum(a.size for a in arrays)
        if total > self.capacity:
            raise ValueError(f"step needs {total} staging words, capacity is {self.capacity}")
        i = self.turn
        self.turn = (i + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        host = self.hosts[i]
        host_np = host.numpy()
        views = []
        off = 0
        for a in arrays:
            host_np[off:off + a.size] = a
            views.append(self.dev[off:off + a.size])
            off += a.size
        if total:
            self.dev[:total].copy_(host[:total], non_blocking=True)
            if self.events[i] is None:
                self.events[i] = torch.cuda.Event()
            self.events[i].record()
        return views


class StepFunction:
    """Builds the batch description, runs the model and keeps the cache's lengths."""

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
        self.buffers = StepBuffers(self.device, max_step_tokens, self.manager.max_slots)
        self.steps_run = 0
        self.graph_launches = 0      # kernels replayed from CUDA graphs (not counted by ops.LAUNCHES)

    # ---- request lifetime ------------------------------------------------------------
    def admit(self, req_id: Hashable) -> None:
        self.manager.admit(req_id)

    def free(self, req_id: Hashable) -> None:
        self.manager.free(req_id)

    def length(self, req_id: Hashable) -> int:
        return self.manager.length(req_id)

    # ---- the step ----------------------------------------------------------------------
    def build(self, entries: Sequence[StepEntry], sampling: Sequence[SamplingRow] | None = None,
              feed: Sequence[int] | None = None) -> tuple[StepBatch, dict]:
        """Reserve pages, lay the batch out and upload its description.

        ``feed`` (with ``sampling`` only) has one number per entry: the place among the previous
        step's sampled tokens whose token is this entry's single token, or -1 for an entry that
        brings its tokens itself."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        tok_parts: list[np.ndarray] = []
        pos_parts: list[np.ndarray] = []
        req_parts: list[np.ndarray] = []
        pf_parts: list[np.ndarray] = []
        q_start: list[int] = []
        q_len: list[int] = []
        kv_len: list[int] = []
        slots: list[int] = []
        rows: list[int] = []
        dec_items: list[int] = []
        n_tokens = 0
        for r, e in enumerate(entries):
            if e.req_id in seen:
                raise ValueError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if not self.manager.has(e.req_id):
                self.admit(e.req_id)
            n = len(e.tokens)
            if n < 1:
                raise ValueError(f"request {e.req_id!r} brings no tokens")
            start = self.manager.length(e.req_id)
            if start + n > self.max_seq_len:
                raise ValueError(f"request {e.req_id!r} would reach {start + n} tokens, "
                                 f"beyond max_seq_len={self.max_seq_len}")
            self.manager.grow(e.req_id, start + n)
            q_start.append(n_tokens)
            q_len.append(n)
            kv_len.append(start + n)
            slots.append(self.manager.slot(e.req_id))
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.req_id!r} wants place {w} of {n} tokens")
                rows.append(n_tokens + w)
            tok_parts.append(np.asarray(e.tokens, dtype=np.int32))
            pos_parts.append(np.arange(start, start + n, dtype=np.int32))
            req_parts.append(np.full(n, r, dtype=np.int32))
            if n == 1:
                dec_items.append(n_tokens)
            else:
                pf_parts.append(np.arange(n_tokens, n_tokens + n, dtype=np.int32))
            n_tokens += n
        if n_tokens > self.max_step_tokens:
            raise ValueError(f"step of {n_tokens} tokens exceeds max_step_tokens={self.max_step_tokens}")
        W = len(rows)
        if sampling is not None and len(sampling) != W:
            raise ValueError(f"{len(sampling)} sampling rows for {W} wanted places")

        i32 = lambda x: np.asarray(x, dtype=np.int32)
        cat = lambda parts: np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)
        arrays = []
        if sampling is not None:
            feed_tok = np.full(n_tokens, -1, dtype=np.int32)
            if feed is not None:
                if len(feed) != len(entries):
                    raise ValueError(f"{len(feed)} feed places for {len(entries)} entries")
                for r, f in enumerate(feed):
                    if f >= 0:
                        if q_len[r] != 1:
                            raise ValueError("only an entry of one token can take it from the previous step")
                        feed_tok[q_start[r]] = f
            seeds = np.asarray([s.seed & 0x7FFFFFFFFFFFFFFF for s in sampling], dtype=np.int64)
            arrays += [seeds.view(np.int32), feed_tok,     # the 64-bit seeds first: they need an even offset
                       np.asarray([s.temperature for s in sampling], dtype=np.float32).view(np.int32),
                       np.asarray([s.top_p for s in sampling], dtype=np.float32).view(np.int32),
                       i32([s.top_k for s in sampling]), i32([s.counter for s in sampling])]

        def tiles_of(rows_per_tile: int) -> list[int]:
            # (request row, tile index) of every request that brings more than one token; tiles
            # with the most keys to visit start first
            tiles = [(kv_len[r] - q_len[r] + rows_per_tile * (t + 1), r, t) for r in range(len(entries))
                     if q_len[r] > 1 for t in range(-(-q_len[r] // rows_per_tile))]
            tiles.sort(reverse=True)
            return [x for _, r, t in tiles for x in (r, t)]

        arrays += [cat(tok_parts), cat(pos_parts), cat(req_parts), i32(q_start), i32(q_len), i32(kv_len),
                   i32(slots), i32(rows), i32(dec_items), cat(pf_parts), i32(tiles_of(64)),
                   i32(tiles_of(ops.PREFILL_TC_ROWS))]
        views = self.buffers.upload(arrays)
        samp = {}
        if sampling is not None:
            samp = {"feed": views[1], "fed": feed is not None,
                    "seed": views[0].view(torch.int64), "temperature": views[2].view(torch.float32),
                    "top_p": views[3].view(torch.float32), "top_k": views[4], "counter": views[5]}
            views = views[6:]
        self.cache.sync()
        batch = StepBatch(
            n_tokens=n_tokens, n_reqs=len(entries), n_want=W,
            token_ids=views[0], positions=views[1], tok_req=views[2], req_q_start=views[3],
            req_q_len=views[4], req_kv_len=views[5], req_slot=views[6], logits_rows=views[7],
            decode_items=views[8], prefill_items=views[9], prefill_tiles=views[10], prefill_tiles_tc=views[11],
            cache=self.cache, err=self.buffers.result[:4],
            host_q_start=q_start, host_q_len=q_len, host_kv_len=kv_len, host_slot=slots,
            max_q_len=max(q_len), max_kv_len=max(kv_len))
        return batch, samp

    def finish(self, entries: Sequence[StepEntry]) -> None:
        """Advance the lengths and give back the pages that a window has passed."""
        for e in entries:
            self.manager.advance(e.req_id, len(e.tokens))
        self.steps_run += 1

    @torch.inference_mode()
    def run(self, entries: Sequence[StepEntry], check: bool = True) -> torch.Tensor:
        """Float32 logits ``[wanted, vocab]`` on the device, in the order of entries and ``want``."""
        batch, _ = self.build(entries)
        logits = self.model.forward(batch)
        self.finish(entries)
        if check:
            self.check_errors()
        return logits

    def run_and_sample(self, entries: Sequence[StepEntry], sampling: Sequence[SamplingRow]) -> list[int]:
        """One token per wanted place, sampled on the device; one copy back for tokens and errors."""
        return self.collect(self.launch_and_sample(entries, sampling))

    @torch.inference_mode()
    def launch_and_sample(self, entries: Sequence[StepEntry], sampling: Sequence[SamplingRow],
                          feed: Sequence[int] | None = None) -> PendingStep:
        """Start a step that samples one token per wanted place on the device; ``collect`` reads them.

        A step in which every request brings exactly one token and wants it sampled has the
        same launches every time, so it is captured into a CUDA graph the second time its shape
        (batch size, bucket of the longest context) is seen and replayed from then on: the
        description of the step is uploaded outside the graph into buffers at fixed addresses.

        With ``feed`` (see ``build``) single tokens come from the previous step's sampled tokens
        on the device, so the step can be launched before that step has been collected: the
        device then never waits for the host between two steps.  At most two launched steps may
        be waiting to be collected, and they are collected in the order of their launch.
        """
        batch, samp = self.build(entries, sampling, feed)
        W = batch.n_want
        res = self.buffers.result
        graphable = (self.use_graphs and batch.max_q_len == 1 and W == batch.n_tokens)
        if graphable:
            bucket = 256
            while bucket < batch.max_kv_len:
                bucket *= 2
            batch.max_kv_len = bucket        # kernels size their grids from the bucket
            key = (batch.n_tokens, bucket)
            graph = self._graphs.get(key)
            if graph is None and self._graph_seen.get(key, 0) >= 1:
                graph = self._capture(key, batch, samp)
            if graph is not None:
                graph["graph"].replay()
                self.graph_launches += graph["kernels"]
            else:
                self._graph_seen[key] = self._graph_seen.get(key, 0) + 1
                graphable = False
        if not graphable:
            if samp["fed"]:
                ops.feed_tokens(batch.token_ids, samp["feed"], res[4:], batch.err)
            logits = self.model.forward(batch)
            if W:
                ops.sample(logits, samp["temperature"], samp["top_k"], samp["top_p"], samp["seed"],
                           samp["counter"], res[4:4 + W])
        self.finish(entries)
        bufs = self.buffers
        host = bufs.result_hosts[bufs.result_turn]
        bufs.result_turn = (bufs.result_turn + 1) % bufs.RING
        host[:4 + W].copy_(res[:4 + W], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return PendingStep(W, host, done)

    def collect(self, pending: PendingStep) -> list[int]:
        """Wait for a launched step and return its sampled tokens; raises on a kernel error."""
        pending.done.synchronize()
        self._raise_on_error(pending.host[:4].tolist())
        return pending.host[4:4 + pending.n_want].tolist()

    def _capture(self, key, batch: StepBatch, samp: dict) -> dict:
        """Record the decode step of this shape; its launches are replayed, not run, here."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        W = batch.n_want
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            # tokens that the previous step sampled (feed >= 0) take their places first
            ops.feed_tokens(batch.token_ids, samp["feed"], self.buffers.result[4:], batch.err)
            logits = self.model.forward(batch)
            ops.sample(logits, samp["temperature"], samp["top_k"], samp["top_p"], samp["seed"],
                       samp["counter"], self.buffers.result[4:4 + W])
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
            raise StepError(f"kernel error {word[0]} ({_ERR_NAMES.get(word[0], 'unknown')}); "
                            f"details {word[1:]}")
