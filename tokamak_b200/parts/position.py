"""Position encodings.  A rotary position part hands the mixer a table of (cos, sin) pairs for
the tokens of the step; the rotation itself happens in the mixer's fused kernel.  An absolute
encoding would instead implement ``add_to_embedding`` (see ``parts/base.py``)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import POSITIONS, Runtime


@dataclass(frozen=True)
class RopeSpec:
    head_dim: int
    theta: float
    kind: str = "rope_neox"


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


@POSITIONS.register("rope_neox")
class RopeNeox:
    """Half-rotation rotary embedding over the whole head
    (src/tokamak/model/layers.py:36-89).

    ``inv_freq[j] = 1 / theta ** (2j / d)`` is formed in float32 from a float32
    ``arange`` exactly as the reference does (layers.py:47); a kernel multiplies it by
    the float32 position and takes cosine and sine in float32, once per step: every
    layer with the same spec reads the same table.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: RopeSpec, tensors: dict, rt: Runtime):
        if spec.head_dim % 2:
            raise ValueError(f"rotary embedding needs an even head_dim, got {spec.head_dim}")
        self.spec = spec
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, spec.head_dim, 2, dtype=torch.float32)
                                         / spec.head_dim))
        self.inv_freq = inv_freq.to(rt.device)

    @staticmethod
    def expected_tensors(spec: RopeSpec) -> dict:
        return {}

    def rotary_table(self, step) -> tuple[torch.Tensor | None, int]:
        """``([tokens, head_dim / 2, 2] float32 of (cos, sin), rotary_dim)`` for the step's tokens."""
        key = ("rope_table", self.spec)
        table = step.scratch.get(key)
        if table is None:
            table = ops.rope_table(step.positions, self.inv_freq)
            step.scratch[key] = table
        return table, self.spec.head_dim


@POSITIONS.register("none")
class NoPosition:
    """No position encoding: queries and keys pass unrotated."""

    GRAPH_SAFE = True

    def __init__(self, spec: NoPositionSpec, tensors: dict, rt: Runtime):
        self.spec = spec

    @staticmethod
    def expected_tensors(spec: NoPositionSpec) -> dict:
        return {}

    def rotary_table(self, step) -> tuple[torch.Tensor | None, int]:
        return None, 0
