"""One generation request as the engine tracks it.

The engine sees a request as one growing token stream (prompt, then what was
generated) with a *cursor*: ``num_computed`` tokens of the stream are in the cache.
Whatever lies between the cursor and the end of the stream is still to be run, in
portions of any size; a step that reaches the end samples the next token.  Preemption
moves the cursor back to 0 and changes nothing else, which is all that recomputation
needs.  The request's random stream is its seed plus the number of tokens generated so
far (the device keeps that count in the request's slot record).

While a step that samples for the request is in flight, the stream has one token more than the
host knows: ``expected`` counts it, so that the step after can be planned, and launched with
that token fed on the device, before the first one's tokens are read.  ``ending`` says that the
token in flight is certainly the last (a length limit), so nothing is planned after it.

The stop rules and their order are the reference's
(src/tokamak/engine/sequence.py:109-127): an end-of-sequence token unless ignored, then
``max_new_tokens``, then the context budget.
"""

from __future__ import annotations

import enum
import random

from ..sampling.params import SamplingParams


class SequenceStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class FinishReason(enum.Enum):
    STOP = "stop"
    LENGTH = "length"


class Sequence:
    """Token stream, cursor and lifecycle of one request."""

    __slots__ = ("seq_id", "sampling_params", "seed", "status", "finish_reason", "num_computed",
                 "num_preemptions", "arrival_time", "first_token_time", "finish_time",
                 "_stream", "_n_prompt", "expected", "ending")

    def __init__(self, seq_id: int, prompt_token_ids: list[int], sampling_params: SamplingParams):
        if len(prompt_token_ids) == 0:
            raise ValueError("prompt_token_ids must not be empty")
        self.seq_id = seq_id
        self.sampling_params = sampling_params
        # an unseeded request draws a seed once, so that recomputation after preemption repeats it
        self.seed = sampling_params.seed if sampling_params.seed is not None else random.getrandbits(62)
        self._stream: list[int] = [int(t) for t in prompt_token_ids]
        self._n_prompt = len(self._stream)
        self.num_computed = 0           # the cursor: tokens of the stream that the cache holds
        self.expected = 0               # tokens that a step in flight samples and the host has not read
        self.ending = False             # the token in flight ends the request for certain
        self.num_preemptions = 0
        self.status = SequenceStatus.WAITING
        self.finish_reason: FinishReason | None = None
        self.arrival_time = self.first_token_time = self.finish_time = None

    # ---- the stream ---------------------------------------------------------------------
    @property
    def num_tokens(self) -> int:
        return len(self._stream)

    @property
    def num_prompt_tokens(self) -> int:
        return self._n_prompt

    @property
    def num_output_tokens(self) -> int:
        return len(self._stream) - self._n_prompt

    @property
    def prompt_token_ids(self) -> list[int]:
        return self._stream[:self._n_prompt]

    @property
    def output_token_ids(self) -> list[int]:
        return self._stream[self._n_prompt:]

    @property
    def num_tokens_due(self) -> int:
        """Length of the stream with the token that a step in flight is sampling."""
        return len(self._stream) + self.expected

    @property
    def num_pending(self) -> int:
        """Tokens between the cursor and the end of the stream (the expected one included)."""
        return len(self._stream) + self.expected - self.num_computed

    def expect_token(self, max_total_tokens: int) -> None:
        """A step that samples for this request has been launched."""
        self.expected = 1
        self.ending = (self.num_output_tokens + 1 >= self.sampling_params.max_new_tokens
                       or len(self._stream) + 1 >= max_total_tokens)

    def tokens_from(self, start: int, count: int) -> list[int]:
        """``count`` tokens of the stream from index ``start``."""
        return self._stream[start:start + count]

    # ---- lifecycle ----------------------------------------------------------------------
    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    def append_output_token(self, token_id: int) -> None:
        if self.is_finished:
            raise RuntimeError(f"Sequence {self.seq_id} is already finished")
        self._stream.append(int(token_id))
        self.expected = 0

    def append_checked(self, token_id: int, *, eos_token_ids: tuple[int, ...],
                       max_total_tokens: int) -> bool:
        """Append a generated token; ``True`` if it ended the request."""
        self.append_output_token(token_id)
        params = self.sampling_params
        reason = None
        if token_id in eos_token_ids and not params.ignore_eos:
            reason = FinishReason.STOP
        elif self.num_output_tokens >= params.max_new_tokens or len(self._stream) >= max_total_tokens:
            reason = FinishReason.LENGTH
        if reason is not None:
            self.finish(reason)
        return reason is not None

    def finish(self, reason: FinishReason) -> None:
        self.status, self.finish_reason = SequenceStatus.FINISHED, reason

    def rewind(self) -> None:
        """Preemption: nothing of the stream is in the cache any more."""
        self.num_computed = 0
        self.expected = 0
        self.num_preemptions += 1
        self.status = SequenceStatus.WAITING

    def __repr__(self) -> str:
        return (f"Sequence({self.seq_id}: {self._n_prompt}+{self.num_output_tokens} tokens, "
                f"cursor {self.num_computed}, {self.status.value})")
