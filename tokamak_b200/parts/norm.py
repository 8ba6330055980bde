"""RMSNorm, fused with the residual sum that precedes it."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import NORMS, OwedNorm, Runtime, TensorReq


@dataclass(frozen=True)
class RMSNormSpec:
    dim: int
    eps: float
    kind: str = "rmsnorm"


@NORMS.register("rmsnorm")
class RMSNorm:
    """``weight * x * rsqrt(mean(x^2) + eps)`` with 32-bit statistics
    (src/tokamak/model/layers.py:16-33).

    The residual stream is float32; ``add_norm`` first adds the pending branch
    output to it (a 32-bit sum) and then normalises the sum, in one kernel.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: RMSNormSpec, name: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = tensors[name]

    @staticmethod
    def expected_tensors(spec: RMSNormSpec, name: str) -> dict[str, TensorReq]:
        return {name: TensorReq((spec.dim,), role="vector")}

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def owed_norm_params(self) -> tuple[torch.Tensor, float] | None:
        """Weight and eps for a product kernel that prepares this norm's input itself."""
        return self.weight, self.spec.eps

    def add_norm(self, resid: torch.Tensor, delta, rows: torch.Tensor | None = None):
        """Normalised rows in the engine's dtype.

        Without ``rows`` the sum ``resid + delta`` is written back to ``resid`` and
        every row is normalised.  With ``rows`` only those rows are summed and
        normalised and ``resid`` is left as it is.  ``delta`` may be an
        :class:`OwedNorm`: the branch has been added to ``resid`` already; if it was
        prepared for this norm it is handed on as it is (its consumer pays the scale).
        """
        if isinstance(delta, OwedNorm):
            if delta.norm is self:
                return delta if rows is None else delta.rows(rows)
            delta = None
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.dim), dtype=self.rt.dtype, device=resid.device)
        ops.add_rmsnorm(resid, delta, self.weight, out, self.spec.eps, rows)
        return out
