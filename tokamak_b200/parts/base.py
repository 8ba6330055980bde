"""What every part of a layer has in common: specs, tensor requests, registries.

A *spec* is a frozen dataclass with a ``kind`` string and the sizes and
constants of one part; it is data, produced by an architecture from its
configuration.  A *part* is the object built from a spec and the weights; it
owns its tensors and calls the kernels.  The registries map ``kind`` to the
class that builds the part, one registry per role:

=============  ==========================================================
role           interface of the registered class
=============  ==========================================================
norm           ``expected_tensors(spec, name)``, ``__init__(spec, name, tensors, rt)``,
               ``add_norm(resid, delta, rows=None) -> normed``
position       ``expected_tensors(spec)``, ``__init__(spec, tensors, rt)`` and one or both of:
               ``rotary_table(step) -> (table | None, rotary_dim)`` with ``table`` float32
               ``[tokens, rotary_dim / 2, 2]`` of (cos, sin) per token, for mixers that rotate
               queries and keys; ``add_to_embedding(resid, step)``, which adds an encoding of
               ``step.positions`` to the float32 residual rows in place (absolute encodings:
               a learned table, sinusoids), for the model's ``embedding_position`` seat
mixer          ``expected_tensors(spec, prefix)``, ``__init__(spec, prefix, tensors, rt)``,
               ``cache_need() -> KVPagesNeed | StateNeed | None``,
               ``forward(h, step, cache_view) -> [N, hidden]``
feed_forward   ``expected_tensors(spec, prefix)``, ``__init__(spec, prefix, tensors, rt)``,
               ``forward(h, step) -> [N, hidden]``
block          ``expected_tensors(spec)``, ``__init__(spec, tensors, rt)``,
               ``cache_need()``, ``forward(resid, pending, step, cache_view) -> (resid, pending)``
embedding      ``expected_tensors(spec)``, ``__init__(spec, tensors, rt)``,
               ``forward(step) -> float32 residual rows [N, hidden]``, attribute ``weight``
head           ``expected_tensors(spec)``, ``__init__(spec, embedding part, tensors, rt)``,
               ``forward(h, step) -> float32 logits [rows, vocab]``
=============  ==========================================================

No part knows which model it is in: it sees its spec, its tensors, the step's
batch description and the view of its own cache.

**Declarations every part may make** (all optional, all read with ``getattr``):

``GRAPH_SAFE = True`` says that the part's ``forward`` launches the same kernels with the same
arguments whatever the step's numbers are: it reads the step through the device tensors of the
batch description only, never through ``step.host_*``, ``step.max_kv_len`` apart (a bucket under
replay), takes no decision on values it would have to read back from the device, and keeps no
host-side state that changes from step to step.  A step of single next tokens is replayed from a
CUDA graph only if every part of the model says so; a model with one part that does not
(the default) runs such steps kernel by kernel, with fresh host values every time.

``weight_bytes()`` returns the bytes of the tensors that one call of the part reads in full
(an embedding table, read by row, reports 0); measurements sum it over the schedule.

``prefill_heads`` (a mixer, or a block on its mixer's behalf) is a hint, not a contract: how many
work items the part makes of one block of prompt tokens (an attention mixer: its query heads).
The step function balances the work list of prompt portions (``step.prefill_tc``) for the smallest
value among the parts; any value gives right results.

**Owed norms.**  In bfloat16 steps of few tokens the kernel of a product that ends a branch can
add its sums to the residual stream itself and hand on the input of the *next* norm with the
scaling by the statistic still owed (:class:`OwedNorm`); the product after that norm pays it in
its epilogue, and the norm between them needs no kernel.  This is opt-in: a mixer or
feed-forward with ``TAKES_THEN_NORM = True`` is called with ``then_norm=(resid, norm part)`` and
may return an :class:`OwedNorm` prepared for that norm instead of its output; one with
``TAKES_OWED_NORM = True`` may be handed an :class:`OwedNorm` as ``h`` (others get a tensor); a
block with ``TAKES_NEXT_NORM = True`` is told which norm will consume what it leaves pending and
names the norm that consumes its own input as ``entry_norm``.  Parts without these attributes
never see any of it.

**Queued products.**  In those same steps the products of consecutive parts (attention output,
gate/up, down, the next block's q|k|v, the head) are not launched one by one: :func:`linear` and the
fused product wrappers queue them in the step's :class:`~tokamak_b200.csrc.ops.ProductChain`
(:func:`chain_of`), and the queue is launched as one persistent kernel when something else needs a
result: every kernel wrapper of ``csrc/ops.py`` flushes it before it launches, and so do
:meth:`OwedNorm.materialize` and the end of the model's forward pass.  Only an :class:`OwedNorm`
carries results across parts that may still be queued, so the rule for a part that opts into owed
norms is: hand its tensors to :func:`linear` or to kernels of this library, or call ``materialize()``;
never read ``xb`` or ``sumsq`` with other code.  A part that passes ``chain=`` to :func:`linear` itself
holds to the same rule for what it gets back.

Where a row says ``[N, hidden]`` a mixer or feed-forward may instead return what
:func:`linear` gave it: a 3-D float32 tensor of partial sums ``[parts, N, hidden]``
from a split-K product.  The norm that consumes it adds the parts up (a 32-bit sum);
:func:`sum_parts` does the same for anyone else.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class TensorReq:
    """A tensor that a part expects in the checkpoint.

    ``role`` decides the element type in memory: ``matrix`` takes the engine's
    dtype; ``vector`` (norm weights and other small per-channel tensors) is held in
    float32, which keeps a tensor stored in 32-bit exact; ``int_table`` becomes int32.
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclass
class Runtime:
    """Where and in which element type the parts live."""

    device: torch.device
    dtype: torch.dtype            # torch.bfloat16 (serving) or torch.float32 (true 32-bit path)

    @property
    def is_f32(self) -> bool:
        return self.dtype == torch.float32


class Registry:
    """Maps the ``kind`` of a spec to the class that builds the part."""

    def __init__(self, role: str) -> None:
        self.role = role
        self._classes: dict[str, Any] = {}

    def register(self, kind: str) -> Callable[[Any], Any]:
        def deco(cls: Any) -> Any:
            if kind in self._classes and self._classes[kind] is not cls:
                raise ValueError(f"{self.role} kind {kind!r} is already registered")
            self._classes[kind] = cls
            return cls
        return deco

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def get(self, kind: str) -> Any:
        try:
            return self._classes[kind]
        except KeyError:
            known = ", ".join(sorted(self._classes)) or "<none>"
            raise KeyError(f"no {self.role} of kind {kind!r} is registered; known: {known}") from None

    def kinds(self) -> list[str]:
        return sorted(self._classes)


NORMS = Registry("norm")
POSITIONS = Registry("position")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed_forward")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")


def graph_safe(*parts: Any) -> bool:
    """Whether every given part declares ``GRAPH_SAFE`` (an attribute, or a method for a part
    made of parts)."""
    for part in parts:
        flag = getattr(part, "GRAPH_SAFE", False)
        if callable(flag):
            flag = flag()
        if not flag:
            return False
    return True


def weight_bytes(*parts: Any) -> int:
    """Sum of ``weight_bytes()`` over the parts that report it."""
    return sum(int(part.weight_bytes()) for part in parts if hasattr(part, "weight_bytes"))


def tensor_bytes(*tensors: Any) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


SWAPPED_GEMM_MAX_TOKENS = 64


@dataclass
class OwedNorm:
    """Input of a norm whose scaling by the statistic is still owed.

    ``xb`` is ``bf16(residual * norm weight)`` (the residual stream already holds the sum),
    ``sumsq`` the sums of squares of the residual rows in tiles ``[tiles, N]``: the normalised
    rows are ``xb * rsqrt(sumsq.sum(0) / dim + eps)``.  ``norm`` is the norm part it was prepared
    for.  :func:`linear` takes it in place of a tensor.
    """

    xb: torch.Tensor
    sumsq: torch.Tensor
    dim: int
    eps: float
    norm: Any

    @property
    def shape(self):
        return self.xb.shape

    @property
    def dtype(self):
        return self.xb.dtype

    @property
    def device(self):
        return self.xb.device

    def materialize(self) -> torch.Tensor:
        """The normalised rows as an ordinary tensor (for a consumer that cannot pay the scale)."""
        from ..csrc import ops
        ops.flush_chains()          # the product that prepares xb and sumsq may still be queued
        rstd = torch.rsqrt(self.sumsq.sum(0) / self.dim + self.eps)
        return (self.xb.float() * rstd[:, None]).to(self.xb.dtype)

    def rows(self, index: torch.Tensor) -> "OwedNorm":
        from ..csrc import ops
        ops.flush_chains()
        return OwedNorm(self.xb.index_select(0, index.long()).contiguous(),
                        self.sumsq.index_select(1, index.long()).contiguous(), self.dim, self.eps, self.norm)


def chain_of(step):
    """The queue of products of a step of few tokens (made on first use), or ``None`` where products
    are launched one by one: no step, more tokens than the chain kernel takes."""
    from ..csrc import ops
    scratch = getattr(step, "scratch", None)
    n = getattr(step, "n_tokens", 0)
    if scratch is None or ops.CHAIN_POLICY != "on" or not ops.ProductChain.takes(n, 128):
        return None
    chain = scratch.get("chain")
    if chain is None:
        chain = scratch["chain"] = ops.ProductChain(n, step.err)
    return chain


def linear(x, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
           err: torch.Tensor | None = None, then_norm: tuple | None = None, chain=None,
           queue_plain: bool = False):
    """``x @ weight^T`` for ``weight`` of shape [out, in].

    float32: the engine's own FFMA kernel (no TF32, no tensor cores).

    bfloat16, few tokens (decoding): the tcgen05 kernel with the weight as the 128-row
    operand, streamed once by TMA and split over K, the splits of a tile added up inside a
    thread-block cluster.  The result is a 3-D float32 tensor ``[parts, tokens, out]`` (one
    or two parts) which the consuming kernel (norm, rotation, activation) adds up; ``err`` is the
    error word its bounded waits report to.  On this path ``x`` may be an :class:`OwedNorm` (the
    kernel multiplies its sums by the owed scale), and with ``then_norm=(resid, norm part)`` the
    kernel adds its sums to the float32 residual stream ``resid`` itself and an :class:`OwedNorm`
    for that norm is returned instead of the product (where the sizes allow it; otherwise the
    product is returned as usual).  With ``chain`` (see :func:`chain_of`) a product that returns an
    :class:`OwedNorm` is queued rather than launched; a product that returns plain sums is launched
    at once (with everything queued before it), so that a tensor handed on to other parts always
    holds its values, unless the caller says ``queue_plain`` and flushes the queue itself.

    bfloat16, many tokens: the persistent tcgen05 kernel on pairs of SMs (``ops.gemm_pair``)
    where its grid fills the GPU; otherwise the library product, as the reference uses the
    library for its projections (src/tokamak/model/transformer.py:38-41); ``out_dtype=float32``
    keeps the 32-bit accumulators instead of rounding them (library only).
    """
    from ..csrc import ops

    if x.dtype == torch.float32:
        return ops.gemm_f32(x, weight)
    if err is not None and x.shape[0] <= SWAPPED_GEMM_MAX_TOKENS and weight.shape[1] % 8 == 0:
        splits, stages, cluster = ops.swapped_gemm_plan(weight.shape[0], weight.shape[1], x.shape[0])
        colscale = None
        if isinstance(x, OwedNorm):
            colscale, x = (x.sumsq, x.dim, x.eps), x.xb
        if then_norm is not None:
            resid, norm = then_norm
            params = norm.owed_norm_params() if hasattr(norm, "owed_norm_params") else None
            if (params is not None and weight.shape[0] % 128 == 0 and resid.dtype == torch.float32
                    and resid.shape == (x.shape[0], weight.shape[0])):
                norm_weight, eps = params
                xb, sumsq = ops.gemm_tc_swapped(weight, x, err, splits, max_stages=stages, cluster=cluster,
                                                colscale=colscale, residual_norm=(resid, norm_weight), chain=chain)
                return OwedNorm(xb, sumsq, weight.shape[0], eps, norm)
        out = ops.gemm_tc_swapped(weight, x, err, splits, max_stages=stages, cluster=cluster, colscale=colscale,
                                  chain=chain)
        if chain is not None and not queue_plain:
            ops.flush_chains()
        return out
    if isinstance(x, OwedNorm):
        x = x.materialize()
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if err is not None and ops.pair_gemm_takes(x.shape[0], weight.shape[0], weight.shape[1]):
        return ops.gemm_pair(x, weight, err)
    return torch.mm(x, weight.t())


def sum_parts(t: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
    """A 2-D tensor from the result of :func:`linear`: partial sums are added up."""
    if t.dim() == 3:
        t = t[0] if t.shape[0] == 1 else t.sum(0)
    return t if dtype is None or t.dtype == dtype else t.to(dtype)
