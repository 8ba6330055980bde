"""Feed-forward parts."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import (FEED_FORWARDS, SWAPPED_GEMM_MAX_TOKENS, OwedNorm, Runtime, TensorReq, chain_of, linear,
                   tensor_bytes)


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@FEED_FORWARDS.register("swiglu")
class SwiGLU:
    """``down(silu(gate(x)) * up(x))`` without biases (src/tokamak/model/layers.py:92-104).

    The gate and up matrices are stacked into one ``[2I, H]`` operand so that one
    product feeds the activation.  Where the intermediate size allows it, their rows
    alternate in blocks of 64 (64 gate rows, then the 64 up rows of the same outputs): a
    128-row tile of the decode product then holds both halves of 64 outputs, and the block
    that adds its K splits up applies the activation itself, so that decoding needs no
    activation kernel and no float32 round trip of the ``[tokens, 2I]`` sums.
    """

    def __init__(self, spec: SwiGLUSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        gate, up = tensors[prefix + "gate_proj.weight"], tensors[prefix + "up_proj.weight"]
        i, h = spec.intermediate_size, spec.hidden_size
        b = ops.SWIGLU_TILE_BLOCK
        if i % b == 0:
            self.block = b
            self.w_gate_up = torch.stack((gate.view(i // b, b, h), up.view(i // b, b, h)), dim=1).reshape(2 * i, h)
        else:
            self.block = i
            self.w_gate_up = torch.cat((gate, up), dim=0)
        self.w_gate_up = self.w_gate_up.contiguous()
        self.w_down = tensors[prefix + "down_proj.weight"]

    @staticmethod
    def expected_tensors(spec: SwiGLUSpec, prefix: str) -> dict[str, TensorReq]:
        h, i = spec.hidden_size, spec.intermediate_size
        return {
            prefix + "gate_proj.weight": TensorReq((i, h)),
            prefix + "up_proj.weight": TensorReq((i, h)),
            prefix + "down_proj.weight": TensorReq((h, i)),
        }

    GRAPH_SAFE = True

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_gate_up, self.w_down)

    TAKES_OWED_NORM = True     # the gate/up product pays an owed norm scale in its epilogue
    TAKES_THEN_NORM = True     # the down product can add itself to the residual stream

    def forward(self, h, step, then_norm=None):
        err = step.err if step is not None else None
        chain = chain_of(step)
        n = h.shape[0]
        if (h.dtype == torch.bfloat16 and err is not None and n <= SWAPPED_GEMM_MAX_TOKENS
                and self.block == ops.SWIGLU_TILE_BLOCK and self.spec.hidden_size % 8 == 0):
            splits, stages, cluster = ops.swapped_gemm_plan(2 * self.spec.intermediate_size, self.spec.hidden_size, n)
            colscale = None
            if isinstance(h, OwedNorm):
                colscale, h = (h.sumsq, h.dim, h.eps), h.xb
            act = ops.gemm_tc_swapped(self.w_gate_up, h, err, splits, max_stages=stages, cluster=cluster,
                                      swiglu=True, colscale=colscale, chain=chain)
        else:
            if isinstance(h, OwedNorm):
                h = h.materialize()
            if (h.dtype == torch.bfloat16 and err is not None and self.block == ops.SWIGLU_TILE_BLOCK
                    and ops.pair_gemm_takes(n, 2 * self.spec.intermediate_size, self.spec.hidden_size, fused=True)):
                # many tokens: the product on pairs of SMs applies the activation to its accumulators
                act = ops.gemm_pair(h, self.w_gate_up, err, swiglu=True)
            else:
                gate_up = linear(h, self.w_gate_up, err=err)
                act = torch.empty((n, self.spec.intermediate_size), dtype=h.dtype, device=h.device)
                ops.swiglu(gate_up, act, block=self.block)
        return linear(act, self.w_down, err=err, then_norm=then_norm, chain=chain)
