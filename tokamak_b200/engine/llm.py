"""The offline batch inference entry point: ``LLM(...).generate(prompts, SamplingParams)``.

Names and meanings of the options follow the reference
(src/tokamak/engine/llm.py:54-122, 265-286).  One ``generate`` call runs a step
loop: the scheduler plans a mixed batch, the step function runs it and samples
on the device, one copy brings the sampled tokens back, and finished requests
give their pages back before the next plan.  Not thread-safe: one ``generate``
call at a time.
"""

from __future__ import annotations

import logging
import time
from pathlib import Path
from typing import Sequence as AbcSequence

import torch

from ..sampling.params import SamplingParams
from .core import EngineCore
from .outputs import RequestOutput
from dataclasses import dataclass

from .scheduler import Scheduler, StepPlan
from .sequence import Sequence
from .step import PendingStep, SamplingRow, StepEntry

logger = logging.getLogger(__name__)


@dataclass
class _Flight:
    """A step that has been launched and not read yet."""

    plan: StepPlan
    pending: PendingStep
    samplers: list          # the sequences that sample in it, in the order of its sampled tokens


def parse_attention_policy(spec: str) -> int | None:
    """``"full"`` or ``"window:W"`` (src/tokamak/model/attention_policy.py:63-86): the window in
    positions, or ``None``.  Sink positions (``streaming:W+S``) are not implemented."""
    if spec == "full":
        return None
    kind, sep, arg = spec.partition(":")
    if sep and kind == "window":
        try:
            window = int(arg)
        except ValueError as err:
            raise ValueError(f"Unknown attention_policy: {spec!r}") from err
        if window < 1:
            raise ValueError(f"window must be >= 1, got {window}")
        return window
    raise ValueError(f"Unknown attention_policy: {spec!r} (expected 'full' or 'window:W')")


def _only(name: str, value, allowed: tuple, why: str) -> None:
    if value not in allowed:
        raise ValueError(f"{name}={value!r} is not available: {why} (allowed: {', '.join(map(repr, allowed))})")


class LLM:
    """Loads a model once and serves batch generation requests.

    Args:
        model: local checkpoint folder (``config.json`` + ``*.safetensors``).
        device: ``"auto"``/``"cuda"`` or an explicit CUDA device; there is no CPU path.
        dtype: ``"auto"``/``"bfloat16"`` or ``"float32"`` (the true 32-bit path).
        max_seq_len: cap on one request's context (prompt + generation); defaults to
            the model's trained maximum.
        block_size: tokens per cache page.
        kv_pool_tokens: token capacity of the page pool; defaults to ``max_seq_len`` and
            must be at least that, so that any single request can finish alone.  ``"auto"``
            (not in the reference) fills ``gpu_memory_utilization`` of the device memory that is
            free after loading, less the measured activations of the largest step.
        gpu_memory_utilization: see ``kv_pool_tokens="auto"``.
        max_batch_size: upper bound on concurrently running sequences.
        max_num_batched_tokens: most tokens of one step (decode tokens plus prompt portions).
        prefill_chunk: most tokens of one prompt portion; ``None`` leaves it to the budget.
        attention_policy: ``"full"`` or ``"window:W"``, a window applied to every layer.
        kv_watermark: share of the page pool that an admission leaves free while other requests
            run (not in the reference; 0 is its behaviour).
        step_token_multiple: a step of more tokens than this is shortened to a multiple of it by
            cutting a prompt portion earlier (not in the reference, whose steps hold whole prompts;
            128 is the token tile of the matrix products; 1 leaves steps as planned).
        kv_backend, scheduling, attention_backend, draft_model, num_speculative_tokens: accepted
            with the reference's defaults (``"paged"``, ``"continuous"``, ``"auto"``, ``None``), so
            that a call written for it still works; any other value is refused with the reason.
    """

    def __init__(self, model: str | Path, *, device: str | torch.device = "auto",
                 dtype: str | torch.dtype = "auto", max_seq_len: int | None = None,
                 block_size: int = 16, kv_pool_tokens: int | str | None = None, max_batch_size: int = 16,
                 max_num_batched_tokens: int = 2048, prefill_chunk: int | None = None,
                 attention_policy: str = "full", gpu_memory_utilization: float = 0.9,
                 kv_watermark: float = 0.0, step_token_multiple: int = 128,
                 kv_backend: str = "paged", scheduling: str = "continuous",
                 attention_backend: str = "auto", draft_model: str | None = None,
                 num_speculative_tokens: int = 4, _core: EngineCore | None = None) -> None:
        # options of the reference whose other values name parts that this engine does not have
        _only("kv_backend", kv_backend, ("paged",), "the cache is always paged")
        _only("scheduling", scheduling, ("continuous",), "requests always join and leave step by step")
        _only("attention_backend", attention_backend, ("auto",), "attention always runs on this engine's kernels")
        if draft_model is not None:
            raise ValueError("draft_model: speculative decoding is not part of this engine")
        if block_size < 1:
            raise ValueError(f"block_size must be >= 1, got {block_size}")
        if max_batch_size < 1:
            raise ValueError(f"max_batch_size must be >= 1, got {max_batch_size}")
        window = parse_attention_policy(attention_policy)
        if _core is not None:
            self.core = _core
        else:
            self.core = EngineCore(model, dtype=dtype, device=device, max_seq_len=max_seq_len,
                                   page_size=block_size, pool_tokens=kv_pool_tokens,
                                   max_slots=max_batch_size,
                                   max_step_tokens=max(max_num_batched_tokens, max_batch_size),
                                   window=window, memory_utilization=gpu_memory_utilization)
        self.model_path = Path(model)
        self.model_config = self.core.config
        self.max_seq_len = self.core.max_seq_len
        self.device = self.core.device
        self.dtype = self.core.dtype
        self.block_size = block_size
        self.max_batch_size = max_batch_size
        self.max_num_batched_tokens = max(max_num_batched_tokens, 1)
        self.prefill_chunk = prefill_chunk
        if not 0.0 <= kv_watermark < 1.0:
            raise ValueError(f"kv_watermark must be in [0, 1), got {kv_watermark}")
        self.kv_watermark = kv_watermark
        if step_token_multiple < 1:
            raise ValueError(f"step_token_multiple must be >= 1, got {step_token_multiple}")
        self.step_token_multiple = step_token_multiple
        self.cache_manager = self.core.manager
        self.model = self.core.model
        self._tokenizer = None
        self.last_stats: dict = {}
        # A debugging aid: with plain_steps every step is laid out by the host (tokens included),
        # none is launched ahead of the one before it and none is replayed from a CUDA graph.  The
        # tokens must not depend on it.
        self.plain_steps = False

    # ---- tokenizer (text in and out only; the engine itself works on token ids) ---------
    @property
    def tokenizer(self):
        if self._tokenizer is None:
            names = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "tokenizer.model")
            if not any((self.model_path / n).is_file() for n in names):
                raise RuntimeError(f"{self.model_path} has no tokenizer files; pass prompt_token_ids")
            from transformers import AutoTokenizer
            self._tokenizer = AutoTokenizer.from_pretrained(self.model_path)
        return self._tokenizer

    def _has_tokenizer(self) -> bool:
        try:
            return self.tokenizer is not None
        except RuntimeError:
            return False

    # ---- generation -------------------------------------------------------------------------
    def generate(self, prompts: str | AbcSequence[str] | None = None,
                 sampling_params: SamplingParams | AbcSequence[SamplingParams] | None = None, *,
                 prompt_token_ids: AbcSequence[AbcSequence[int]] | None = None,
                 use_tqdm: bool = False) -> list[RequestOutput]:
        """Generate a completion for each prompt; one ``RequestOutput`` per prompt, in input order.

        Exactly one of ``prompts`` and ``prompt_token_ids`` is given.  ``sampling_params`` is one
        object for all prompts, a sequence matching them one to one, or ``None`` for defaults.
        """
        texts, token_lists = self._token_lists(prompts, prompt_token_ids)
        per_prompt = self._params_per_prompt(sampling_params, len(token_lists))

        arrival = time.perf_counter()
        sequences = []
        for i, (ids, params) in enumerate(zip(token_lists, per_prompt, strict=True)):
            seq = Sequence(seq_id=i, prompt_token_ids=ids, sampling_params=params)
            seq.arrival_time = arrival
            self._check_request(seq)
            sequences.append(seq)

        scheduler = Scheduler(self.cache_manager, self.max_batch_size, self.max_num_batched_tokens,
                              self.prefill_chunk, self.kv_watermark, self.step_token_multiple)
        for seq in sequences:
            scheduler.add(seq)

        bar = None
        if use_tqdm:
            from tqdm.auto import tqdm
            bar = tqdm(total=len(sequences), desc="Generating")
        buffers = self.core.step.buffers
        stats = {"steps": 0, "tokens_run": 0, "prefill_tokens": 0, "decode_tokens": 0,
                 "mixed_steps": 0, "decode_steps": 0, "decode_step_time_s": 0.0,
                 "steps_launched_ahead": 0, "portions_launched_ahead": 0,
                 "decode_step_tokens": 0, "decode_step_times": [], "decode_step_h2d_bytes": [],
                 "pages_free_min": min((g.num_free for g in self.cache_manager.kv_groups), default=0)}
        try:
            flight = None                    # the launched step whose tokens have not been read
            mark = time.perf_counter()       # when the device last became free for a new step
            h2d_mark = buffers.h2d_bytes
            while flight is not None or scheduler.has_unfinished():
                if flight is None:
                    mark = time.perf_counter()
                    plan = scheduler.schedule()
                    if plan is None:
                        raise RuntimeError("scheduler returned no work but is unfinished")
                    flight = self._launch(plan)
                # the step after this one is known but for the tokens that this one samples, and
                # those stay on the device: it is launched before this step's tokens are read
                ahead = None
                plan_ahead = None if self.plain_steps else scheduler.plan_ahead(flight.plan, self._context_budget)
                if plan_ahead is not None:
                    ahead = self._launch(plan_ahead)
                    stats["steps_launched_ahead"] += 1
                    stats["portions_launched_ahead"] += sum(1 for e in plan_ahead.entries if e.count > 1)
                done = self._complete(flight, ahead)
                plan = flight.plan
                stats["steps"] += 1
                stats["tokens_run"] += plan.num_tokens
                n_dec = sum(1 for e in plan.entries if e.count == 1 and e.start > 0)
                stats["decode_tokens"] += n_dec
                stats["prefill_tokens"] += plan.num_tokens - n_dec
                stats["mixed_steps"] += int(0 < n_dec < len(plan.entries))
                stats["pages_free_min"] = min([stats["pages_free_min"]]
                                              + [g.num_free for g in self.cache_manager.kv_groups])
                now = time.perf_counter()
                if n_dec == len(plan.entries):
                    # a step of single next tokens only, timed from the moment the device was free
                    # for it (planning, or the end of the step before it) to its tokens on the host
                    dt = now - mark
                    stats["decode_steps"] += 1
                    stats["decode_step_time_s"] += dt
                    stats["decode_step_tokens"] += n_dec
                    stats["decode_step_times"].append(dt)
                    # bytes copied to the device since the step before was accounted for
                    stats["decode_step_h2d_bytes"].append(buffers.h2d_bytes - h2d_mark)
                h2d_mark = buffers.h2d_bytes
                mark = now
                if bar is not None:
                    bar.update(done)
                flight = ahead
        finally:
            for seq in sequences:
                self.cache_manager.free(seq.seq_id)
            if bar is not None:
                bar.close()
        stats["preemptions"] = scheduler.num_preemptions
        stats["pages_free"] = [g.num_free for g in self.cache_manager.kv_groups]
        self.last_stats = stats
        return [self._result_of(seq, texts[seq.seq_id] if texts else None) for seq in sequences]

    def _launch(self, plan: StepPlan) -> "_Flight":
        """Start one planned step.

        A request that was given a slot in this plan gets its record written: how it samples, its
        seed, a counter of zero.  A request that only needs its next token does not bring it: the
        device sampled it and holds it in the request's record, whether or not the host has read
        it yet."""
        entries, samplers = [], []
        for seq in plan.admitted:
            p = seq.sampling_params
            self.core.step.set_record(seq.seq_id, SamplingRow(p.temperature, p.top_k, p.top_p, seq.seed, 0),
                                      fresh=True)
        for e in plan.entries:
            seq = e.seq
            # its last sampled token: known to the host or, in a step planned ahead, still to be read
            on_device = (e.count == 1 and e.samples and not self.plain_steps
                         and (seq.num_output_tokens > 0 or e.start >= seq.num_tokens))
            tokens = None if on_device else seq.tokens_from(e.start, e.count)
            if tokens is not None and len(tokens) != e.count:
                raise RuntimeError(f"sequence {seq.seq_id}: tokens {e.start}..{e.start + e.count} are not all known")
            entries.append(StepEntry(seq.seq_id, tokens, [e.count - 1] if e.samples else []))
            if e.samples:
                samplers.append(seq)
            seq.num_computed = e.start + e.count
        step = self.core.step
        graphs, step.use_graphs = step.use_graphs, step.use_graphs and not self.plain_steps
        try:
            pending = step.launch_and_sample(entries)
        finally:
            step.use_graphs = graphs
        return _Flight(plan, pending, samplers)

    def _complete(self, flight: "_Flight", ahead: "_Flight | None") -> int:
        """Read a step's tokens, append them and free what finished."""
        tokens = self.core.step.collect(flight.pending)
        now = time.perf_counter()
        in_ahead = {id(s) for s in ahead.samplers} if ahead is not None else set()
        finished = 0
        for seq, token in zip(flight.samplers, tokens):
            if seq.is_finished:
                # it stopped in the step before, while this one was already running
                self.cache_manager.free(seq.seq_id)
                continue
            done = seq.append_checked(int(token), eos_token_ids=self.model_config.eos_token_ids,
                                      max_total_tokens=self._context_budget(seq))
            if seq.first_token_time is None:
                seq.first_token_time = now
            if done:
                seq.finish_time = now
                finished += 1
                if id(seq) not in in_ahead:
                    self.cache_manager.free(seq.seq_id)
        return finished

    # ---- what a request may ask for --------------------------------------------------------------
    def _context_budget(self, seq: Sequence) -> int:
        """Tokens the request's stream may reach: its own limit or the engine's, whichever is less."""
        return min(seq.num_prompt_tokens + seq.sampling_params.max_new_tokens, self.max_seq_len)

    def _check_request(self, seq: Sequence) -> None:
        """Refuse at submission what could never run: a prompt that leaves no room to generate,
        token ids the embedding does not have, more pages than the whole pool."""
        n, vocab = seq.num_prompt_tokens, self.model_config.vocab_size
        if n >= self.max_seq_len:
            raise ValueError(f"a prompt of {n} tokens does not fit: max_seq_len={self.max_seq_len} must "
                             f"leave room for at least one generated token")
        for t in seq.prompt_token_ids:
            if not 0 <= t < vocab:
                raise ValueError(f"prompt token id {t} is outside the vocabulary of {vocab}")
        budget = self._context_budget(seq)
        for g in self.cache_manager.kv_groups:
            need = g.pages_for(budget)
            if need > g.num_pages:
                raise ValueError(f"the request needs {need} cache pages at its longest and the pool has "
                                 f"{g.num_pages}: raise kv_pool_tokens")

    def _token_lists(self, prompts, prompt_token_ids) -> tuple[list[str] | None, list[list[int]]]:
        """Texts (if prompts came as text) and the token ids of every prompt."""
        given = [x is not None for x in (prompts, prompt_token_ids)]
        if sum(given) != 1:
            raise ValueError("give exactly one of `prompts` (text) and `prompt_token_ids`")
        if prompt_token_ids is not None:
            return None, [[int(t) for t in ids] for ids in prompt_token_ids]
        texts = [prompts] if isinstance(prompts, str) else list(prompts)
        encode = self.tokenizer.encode
        return texts, [encode(text) for text in texts]

    def _result_of(self, seq: Sequence, prompt_text: str | None) -> RequestOutput:
        if not seq.is_finished:
            raise RuntimeError(f"request {seq.seq_id} left the step loop unfinished")
        since = lambda t: None if t is None or seq.arrival_time is None else t - seq.arrival_time
        generated = seq.output_token_ids
        text = ""
        if self._has_tokenizer():
            decode = self.tokenizer.decode
            text = decode(generated, skip_special_tokens=True)
            if prompt_text is None:
                prompt_text = decode(seq.prompt_token_ids, skip_special_tokens=True)
        return RequestOutput(request_id=seq.seq_id, prompt=prompt_text,
                             prompt_token_ids=seq.prompt_token_ids, output_text=text,
                             output_token_ids=generated, finish_reason=seq.finish_reason,
                             ttft_s=since(seq.first_token_time), latency_s=since(seq.finish_time),
                             num_preemptions=seq.num_preemptions)

    @staticmethod
    def _params_per_prompt(sampling_params, n: int) -> list[SamplingParams]:
        if isinstance(sampling_params, SamplingParams) or sampling_params is None:
            return [sampling_params or SamplingParams()] * n
        per_prompt = list(sampling_params)
        if len(per_prompt) != n:
            raise ValueError(f"{len(per_prompt)} SamplingParams for {n} prompts: give one, or one each")
        return per_prompt
