"""Arrangements of a mixer, a feed-forward and their norms in one block."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, OwedNorm, Runtime, TensorReq, graph_safe, weight_bytes


@dataclass(frozen=True)
class PreNormBlockSpec:
    """One block and the checkpoint names of its tensors.

    ``mixer_prefix`` and ``ffn_prefix`` end with a dot; ``norm1_name`` and
    ``norm2_name`` are full tensor names.
    """

    name: str
    norm1: object
    mixer: object
    norm2: object
    feed_forward: object
    norm1_name: str
    mixer_prefix: str
    norm2_name: str
    ffn_prefix: str
    kind: str = "pre_norm"


@BLOCKS.register("pre_norm")
class PreNormBlock:
    """``x = x + mixer(norm1(x)); x = x + ffn(norm2(x))``
    (src/tokamak/model/transformer.py:89-109).

    The block receives the float32 residual stream and the branch output that
    has not been added to it yet; each norm call adds the pending branch and
    normalises the sum in one kernel.  The second branch's output is returned as
    the new pending value, to be added by whoever normalises next.

    Where a branch can, its last product adds itself to the residual stream and prepares
    the input of the norm after it (see ``parts/base.py``, owed norms): the mixer for
    ``norm2``, the feed-forward for ``next_norm``, the norm that will consume what this
    block leaves pending.
    """

    TAKES_NEXT_NORM = True

    def __init__(self, spec: PreNormBlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, spec.norm1_name, tensors, rt)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.mixer_prefix, tensors, rt)
        self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, spec.norm2_name, tensors, rt)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
            spec.feed_forward, spec.ffn_prefix, tensors, rt)

    @staticmethod
    def expected_tensors(spec: PreNormBlockSpec) -> dict[str, TensorReq]:
        out: dict[str, TensorReq] = {}
        out.update(NORMS.get(spec.norm1.kind).expected_tensors(spec.norm1, spec.norm1_name))
        out.update(MIXERS.get(spec.mixer.kind).expected_tensors(spec.mixer, spec.mixer_prefix))
        out.update(NORMS.get(spec.norm2.kind).expected_tensors(spec.norm2, spec.norm2_name))
        out.update(FEED_FORWARDS.get(spec.feed_forward.kind).expected_tensors(
            spec.feed_forward, spec.ffn_prefix))
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.norm1, self.mixer, self.norm2, self.feed_forward)

    @property
    def prefill_heads(self) -> int | None:
        """The mixer's hint for the work list of prompt portions, if it gives one."""
        return getattr(self.mixer, "prefill_heads", None)

    def weight_bytes(self) -> int:
        return weight_bytes(self.norm1, self.mixer, self.norm2, self.feed_forward)

    @property
    def entry_norm(self):
        return self.norm1

    @staticmethod
    def _branch(part, h, args: tuple, then_norm):
        if isinstance(h, OwedNorm) and not getattr(part, "TAKES_OWED_NORM", False):
            h = h.materialize()
        if then_norm is not None and getattr(part, "TAKES_THEN_NORM", False):
            return part.forward(h, *args, then_norm=then_norm)
        return part.forward(h, *args)

    def forward(self, resid: torch.Tensor, pending, step, cache_view, next_norm=None):
        h = self.norm1.add_norm(resid, pending)
        a = self._branch(self.mixer, h, (step, cache_view), (resid, self.norm2))
        h = self.norm2.add_norm(resid, a)
        out = self._branch(self.feed_forward, h, (step,), (resid, next_norm) if next_norm is not None else None)
        return resid, out
