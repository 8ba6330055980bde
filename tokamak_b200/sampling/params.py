"""User-facing sampling configuration; names, defaults and checks of the reference
(src/tokamak/sampling_params.py:6-46)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True, slots=True)
class SamplingParams:
    """Parameters controlling token sampling for a single request.

    Filters apply in the order temperature, top-k, top-p.

    Attributes:
        temperature: softmax temperature; ``0.0`` selects greedy decoding.
        top_k: sample only from the ``top_k`` most likely tokens; ``0`` disables.
        top_p: nucleus sampling, ``1.0`` disables.
        max_new_tokens: hard cap on the number of generated tokens.
        seed: per-request seed; the i-th sampled token of a request with a seed
            depends on (seed, i) only, not on batching or preemption.  ``None``
            draws a seed from Python's global generator when the request is made.
        ignore_eos: keep generating past EOS until another stop condition hits.
    """

    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    max_new_tokens: int = 128
    seed: int | None = None
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.max_new_tokens < 1:
            raise ValueError(f"max_new_tokens must be >= 1, got {self.max_new_tokens}")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0
