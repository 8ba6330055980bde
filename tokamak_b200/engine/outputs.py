"""Result record of one request (src/tokamak/engine/outputs.py:12-38)."""

from __future__ import annotations

from dataclasses import dataclass

from .sequence import FinishReason


@dataclass(frozen=True, slots=True)
class RequestOutput:
    """Completed generation for one prompt.

    ``output_token_ids`` includes a final EOS if one was generated; ``ttft_s`` and
    ``latency_s`` count from submission; ``num_preemptions`` says how often the
    request lost its pages and was recomputed.
    """

    request_id: int
    prompt: str | None
    prompt_token_ids: list[int]
    output_text: str
    output_token_ids: list[int]
    finish_reason: FinishReason
    ttft_s: float | None = None
    latency_s: float | None = None
    num_preemptions: int = 0
