"""Per-request token state (src/tokamak/engine/sequence.py:17-138), with the count of
tokens that the cache already holds, which chunked prefill needs."""

from __future__ import annotations

import enum
import random

from ..sampling.params import SamplingParams


class SequenceStatus(enum.Enum):
    WAITING = enum.auto()
    RUNNING = enum.auto()
    FINISHED = enum.auto()


class FinishReason(enum.Enum):
    STOP = "stop"        # an EOS token was generated
    LENGTH = "length"    # max_new_tokens or the context limit was reached


class Sequence:
    """Tokens and lifecycle of one generation request.

    A preempted sequence goes back to WAITING with its generated tokens intact
    and ``num_computed`` reset; resuming recomputes the cache over prompt plus
    generated tokens, in portions, and then samples the next token.
    """

    def __init__(self, seq_id: int, prompt_token_ids: list[int], sampling_params: SamplingParams):
        if not prompt_token_ids:
            raise ValueError("prompt_token_ids must not be empty")
        self.seq_id = seq_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.output_token_ids: list[int] = []
        self.sampling_params = sampling_params
        self.status = SequenceStatus.WAITING
        self.finish_reason: FinishReason | None = None
        self.arrival_time: float | None = None
        self.first_token_time: float | None = None
        self.finish_time: float | None = None
        self.num_computed = 0
        self.num_preemptions = 0
        seed = sampling_params.seed
        self.seed = seed if seed is not None else random.getrandbits(62)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def tokens_from(self, start: int, count: int) -> list[int]:
        """``count`` tokens of prompt + generated, beginning at index ``start``."""
        n_prompt = len(self.prompt_token_ids)
        end = start + count
        if end <= n_prompt:
            return self.prompt_token_ids[start:end]
        if start >= n_prompt:
            return self.output_token_ids[start - n_prompt:end - n_prompt]
        return self.prompt_token_ids[start:] + self.output_token_ids[:end - n_prompt]

    @property
    def last_token_id(self) -> int:
        return self.output_token_ids[-1] if self.output_token_ids else self.prompt_token_ids[-1]

    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    def append_output_token(self, token_id: int) -> None:
        if self.is_finished:
            raise RuntimeError(f"Sequence {self.seq_id} is already finished")
        self.output_token_ids.append(token_id)

    def append_checked(self, token_id: int, *, eos_token_ids: tuple[int, ...],
                       max_total_tokens: int) -> bool:
        """Append one token and apply the stop rules in the reference's order: EOS unless
        ignored, then ``max_new_tokens``, then the context budget (sequence.py:109-127)."""
        self.append_output_token(token_id)
        params = self.sampling_params
        if not params.ignore_eos and token_id in eos_token_ids:
            self.finish(FinishReason.STOP)
        elif self.num_output_tokens >= params.max_new_tokens or self.num_tokens >= max_total_tokens:
            self.finish(FinishReason.LENGTH)
        return self.is_finished

    def finish(self, reason: FinishReason) -> None:
        self.status = SequenceStatus.FINISHED
        self.finish_reason = reason

    def __repr__(self) -> str:
        return (f"Sequence(id={self.seq_id}, prompt={self.num_prompt_tokens} tok, "
                f"output={self.num_output_tokens} tok, computed={self.num_computed}, "
                f"status={self.status.name})")
