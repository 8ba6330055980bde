"""Position encodings.  A position part hands the mixer a table of rotation
frequencies; the rotation itself happens in the mixer's fused kernel."""

from __future__ import annotations

from dataclasses import dataclass

import torch

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
    ``arange`` exactly as the reference does (layers.py:47); the kernel multiplies
    it by the float32 position and takes sine and cosine in float32.
    """

    def __init__(self, spec: RopeSpec, rt: Runtime):
        if spec.head_dim % 2:
            raise ValueError(f"rotary embedding needs an even head_dim, got {spec.head_dim}")
        self.spec = spec
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, spec.head_dim, 2, dtype=torch.float32)
                                         / spec.head_dim))
        self.inv_freq = inv_freq.to(rt.device)

    def rotary_table(self) -> tuple[torch.Tensor | None, int]:
        return self.inv_freq, self.spec.head_dim


@POSITIONS.register("none")
class NoPosition:
    """No position encoding: queries and keys pass unrotated."""

    def __init__(self, spec: NoPositionSpec, rt: Runtime):
        self.spec = spec

    def rotary_table(self) -> tuple[torch.Tensor | None, int]:
        return None, 0
