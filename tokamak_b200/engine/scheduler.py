"""Iteration-level scheduler: admits requests, cuts prompts into portions, decodes, frees.

Policy of the reference (src/tokamak/engine/scheduler.py:1-188): first come first
served, requests join and leave at token granularity, and when the page pool
cannot cover a running sequence's next tokens the newest running sequence is
preempted: its pages are given back and it returns to the *front* of the waiting
queue with its generated tokens kept, to be recomputed later.  It keeps its request
slot meanwhile, and with it the record of its random generator, as the reference keeps
a preempted request's generator (src/tokamak/engine/llm.py:339-340,441-445); since
nobody is admitted ahead of it, the slot would have no other taker.

What is added here is the token budget, and the rounding of a step's size.  The reference computes a whole prompt
in one step and lets the decodes wait meanwhile (scheduler.py:114-117); this
scheduler plans one mixed batch per step: every running sequence that only needs
its next token gets one token, and what is left of ``max_num_batched_tokens``
goes to prompt portions, running prefills first, then new admissions, each
portion at most ``prefill_chunk`` tokens.  With ``token_multiple`` m > 1 a step of more than m
tokens is then shortened to a multiple of m by cutting a portion that does not end its prompt (it can
be cut anywhere): the matrix products run in tiles of 128 tokens, so 536 tokens cost five tiles and
512 cost four, and the tokens left out come first in the next step.

Order within a plan: the running sequences reserve the pages of their next tokens first, and
admissions take what is left.  The reference asks the admission question first and finds the
running sequences' pages afterwards (scheduler.py:113-131), so it can admit a request whose
pages the next step takes away again; here a request is admitted only into room that the
running sequences leave in this very step.

When pages run out:
  * a waiting request is admitted only if the pages for all its current tokens
    are free now (scheduler.py:144-148); they are reserved at admission;
  * a running sequence that needs a page which is not free preempts the newest
    running sequence (possibly itself) and tries again (scheduler.py:162-188);
  * a request alone in an empty pool that still does not fit is an error, which
    the engine rules out at submission.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager, OutOfPagesError
from .sequence import Sequence, SequenceStatus


@dataclass
class PlannedEntry:
    """Tokens ``[start, start + count)`` of a sequence run this step; ``samples`` says
    that they end at its last known token, so the step samples the next one."""

    seq: Sequence
    start: int
    count: int
    samples: bool


@dataclass
class StepPlan:
    entries: list[PlannedEntry]
    preempted: list[Sequence] = field(default_factory=list)
    admitted: list[Sequence] = field(default_factory=list)    # given a slot for the first time in this plan

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    """FCFS scheduler with a per-step token budget and preemption by recomputation.

    Args:
        manager: the cache manager to reserve pages and slots from.
        max_batch_size: most sequences running at a time.
        max_num_batched_tokens: most tokens of one step.
        prefill_chunk: most tokens of one sequence's prompt portion in a step
            (``None``: limited by the budget only).
        token_multiple: a step of more tokens than this is cut down to a multiple of it where a
            prompt portion allows (1: steps are left as planned).
        watermark: share of every pool that an admission must leave free while other sequences
            run, as room for their growth (fewer preemptions at the price of later admissions).
            The reference has none (docs/design/003-continuous-batching.md:59-62), which is the
            default; a request that is alone is admitted whenever it fits.
    """

    def __init__(self, manager: CacheManager, max_batch_size: int, max_num_batched_tokens: int,
                 prefill_chunk: int | None = None, watermark: float = 0.0, token_multiple: int = 1):
        if max_batch_size < 1:
            raise ValueError(f"max_batch_size must be >= 1, got {max_batch_size}")
        if max_num_batched_tokens < 1:
            raise ValueError(f"max_num_batched_tokens must be >= 1, got {max_num_batched_tokens}")
        if prefill_chunk is not None and prefill_chunk < 1:
            raise ValueError(f"prefill_chunk must be >= 1, got {prefill_chunk}")
        if token_multiple < 1:
            raise ValueError(f"token_multiple must be >= 1, got {token_multiple}")
        if not 0.0 <= watermark < 1.0:
            raise ValueError(f"watermark must be in [0, 1), got {watermark}")
        if max_batch_size > manager.max_slots:
            raise ValueError(f"max_batch_size ({max_batch_size}) exceeds the cache's request "
                             f"slots ({manager.max_slots})")
        self._manager = manager
        self._max_batch_size = max_batch_size
        self._budget = max_num_batched_tokens
        self._chunk = prefill_chunk
        self._watermark = watermark
        self._multiple = token_multiple
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0

    def add(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting) or any(not s.is_finished for s in self.running)

    # ------------------------------------------------------------------------------
    def schedule(self) -> StepPlan | None:
        """Plan the next step; ``None`` when everything is finished."""
        return self._plan(ahead=False)

    def _plan(self, ahead: bool) -> StepPlan | None:
        """The next step.  ``ahead``: a step is in flight whose tokens are not known; sequences that
        it samples for count one token more (``Sequence.expected``), those that it certainly ends
        are left alone, and where the plan would need a preemption, or has nothing to run, the
        answer is ``None``: that is decided once the step in flight has been read."""
        self.running = [s for s in self.running if not s.is_finished]
        preempted: list[Sequence] = []
        admitted: list[Sequence] = []
        while True:
            entries: list[PlannedEntry] = []
            budget = self._budget

            # 1. running sequences: single next tokens first, then prompt portions
            going = [s for s in self.running if not (ahead and s.ending)]
            decoding = [s for s in going if s.num_pending == 1]
            prefilling = [s for s in going if s.num_pending > 1]
            for seq in decoding + prefilling:
                if seq not in self.running:
                    continue    # preempted while an earlier sequence was served
                if budget == 0:
                    break
                want = seq.num_pending
                count = min(want, budget, self._chunk or want)
                if ahead:
                    try:
                        self._manager.grow(seq.seq_id, seq.num_computed + count)
                    except OutOfPagesError:
                        return None     # somebody has to give way: not decided ahead
                elif not self._reserve(seq, seq.num_computed + count, preempted, entries):
                    continue
                entries.append(PlannedEntry(seq, seq.num_computed, count,
                                            samples=seq.num_computed + count == seq.num_tokens_due))
                budget -= count
            # sequences that were preempted after they had been planned drop out
            entries = [e for e in entries if e.seq in self.running]

            # 2. admissions, strictly in arrival order
            while self.waiting and len(self.running) < self._max_batch_size and budget > 0:
                seq = self.waiting[0]
                resumed = self._manager.has(seq.seq_id)     # preempted earlier: it kept its slot
                if (not resumed and self._manager.num_free_slots == 0) or not self._fits_new(seq):
                    if not self.running and not ahead:
                        raise OutOfPagesError(
                            f"sequence {seq.seq_id} needs more pages than the pool can ever provide")
                    break   # pages are busy; decode until some come free
                self.waiting.popleft()
                if not resumed:
                    self._manager.admit(seq.seq_id)
                    admitted.append(seq)
                self._manager.grow(seq.seq_id, seq.num_tokens)
                seq.status = SequenceStatus.RUNNING
                seq.num_computed = 0
                self.running.append(seq)
                count = min(seq.num_tokens, budget, self._chunk or seq.num_tokens)
                entries.append(PlannedEntry(seq, 0, count, samples=count == seq.num_tokens))
                budget -= count

            if entries:
                self._round_down(entries)
                return StepPlan(entries, preempted, admitted)
            if ahead:
                return None
            if self.running:
                # unreachable: a running sequence is either planned or preempted above
                raise RuntimeError("scheduler stalled with running sequences")
            if self.waiting:
                continue
            return None

    def _round_down(self, entries: list[PlannedEntry]) -> None:
        """Shorten the plan to a multiple of ``token_multiple`` tokens, if it has more than that and a
        portion that does not end its prompt can give the remainder up (the latest such portion
        does; pages reserved for the tokens left out are kept for the next step)."""
        total = sum(e.count for e in entries)
        rest = total % self._multiple
        if total <= self._multiple or rest == 0:
            return
        for e in reversed(entries):
            if not e.samples and e.count > rest:
                e.count -= rest
                return

    def plan_ahead(self, plan: StepPlan, max_total_tokens) -> StepPlan | None:
        """The step after ``plan``, decided while ``plan`` is in flight and its tokens are not known
        yet, or ``None``.

        Every sequence that ``plan`` samples for brings one more token, which only the device
        knows; sequences that reach a length limit with it (``max_new_tokens``, or
        ``max_total_tokens(seq)``) are left out, and so are their pages: they are freed when
        ``plan`` has been read.  Prompt portions go on, and requests are admitted into the room
        that is free now.  A sequence that turns out to have stopped on an end-of-sequence token in
        ``plan`` is in the step for nothing; the engine throws its token away.  When pages are short
        the answer is ``None``: who gives way is decided by ``schedule`` once ``plan`` has been read.
        """
        for e in plan.entries:
            if e.samples and not e.seq.is_finished:
                e.seq.expect_token(max_total_tokens(e.seq))
        return self._plan(ahead=True)

    # ------------------------------------------------------------------------------
    def _fits_new(self, seq: Sequence) -> bool:
        keep = self._watermark if self.running else 0.0
        return all(g.pages_for(seq.num_tokens) + int(keep * g.num_pages) <= g.num_free
                   for g in self._manager.kv_groups)

    def _reserve(self, seq: Sequence, num_tokens: int, preempted: list[Sequence],
                 entries: list[PlannedEntry]) -> bool:
        """Pages for ``num_tokens`` positions of a running sequence, preempting on demand."""
        while True:
            try:
                self._manager.grow(seq.seq_id, num_tokens)
                return True
            except OutOfPagesError:
                victim = self.running[-1]   # newest arrival = lowest priority
                self._preempt(victim)
                preempted.append(victim)
                if victim is seq:
                    return False

    def _preempt(self, victim: Sequence) -> None:
        """Evict by recomputation: give back the pages, keep the slot, requeue at the front."""
        self._manager.restart(victim.seq_id)
        self.running.remove(victim)
        victim.rewind()
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
