"""Feed-forward parts."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import FEED_FORWARDS, Runtime, TensorReq, linear


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@FEED_FORWARDS.register("swiglu")
class SwiGLU:
    """``down(silu(gate(x)) * up(x))`` without biases (src/tokamak/model/layers.py:92-104).

    The gate and up matrices are stacked into one ``[2I, H]`` operand so that one
    product feeds the activation kernel.
    """

    def __init__(self, spec: SwiGLUSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.w_gate_up = torch.cat((tensors[prefix + "gate_proj.weight"],
                                    tensors[prefix + "up_proj.weight"]), dim=0).contiguous()
        self.w_down = tensors[prefix + "down_proj.weight"]

    @staticmethod
    def expected_tensors(spec: SwiGLUSpec, prefix: str) -> dict[str, TensorReq]:
        h, i = spec.hidden_size, spec.intermediate_size
        return {
            prefix + "gate_proj.weight": TensorReq((i, h)),
            prefix + "up_proj.weight": TensorReq((i, h)),
            prefix + "down_proj.weight": TensorReq((h, i)),
        }

    def forward(self, h: torch.Tensor, step) -> torch.Tensor:
        err = step.err if step is not None else None
        gate_up = linear(h, self.w_gate_up, err=err)
        act = torch.empty((h.shape[0], self.spec.intermediate_size), dtype=h.dtype, device=h.device)
        ops.swiglu(gate_up, act)
        return linear(act, self.w_down, err=err)
