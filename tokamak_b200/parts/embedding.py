"""Token embedding and the output head."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import EMBEDDINGS, HEADS, Runtime, TensorReq, chain_of, linear, sum_parts, tensor_bytes


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    name: str = "model.embed_tokens.weight"
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Output projection; ``tied`` reuses the embedding table
    (src/tokamak/model/transformer.py:154-156)."""

    vocab_size: int
    hidden_size: int
    tied: bool
    name: str = "lm_head.weight"
    kind: str = "linear_head"


@EMBEDDINGS.register("embedding")
class Embedding:
    """Row lookup without scaling (src/tokamak/model/transformer.py:140); the rows
    are widened into the float32 residual stream."""

    GRAPH_SAFE = True

    def weight_bytes(self) -> int:
        return 0          # read by row: a step touches one row per token

    def __init__(self, spec: EmbeddingSpec, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.weight = tensors[spec.name]

    @staticmethod
    def expected_tensors(spec: EmbeddingSpec) -> dict[str, TensorReq]:
        return {spec.name: TensorReq((spec.vocab_size, spec.hidden_size))}

    def forward(self, step) -> torch.Tensor:
        resid = torch.empty((step.n_tokens, self.spec.hidden_size), dtype=torch.float32,
                            device=self.weight.device)
        ops.embed_gather(self.weight, step.token_ids, resid, step.err)
        return resid


@HEADS.register("linear_head")
class Head:
    """Logits in float32 for the rows that were asked for
    (src/tokamak/model/transformer.py:173-176).  In bfloat16 the product keeps its
    32-bit accumulators rather than rounding them to bfloat16 first."""

    GRAPH_SAFE = True
    TAKES_OWED_NORM = True     # the product pays an owed norm scale in its epilogue

    def weight_bytes(self) -> int:
        return tensor_bytes(self.weight)

    def __init__(self, spec: HeadSpec, embedding, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.weight = embedding.weight if spec.tied else tensors[spec.name]

    @staticmethod
    def expected_tensors(spec: HeadSpec) -> dict[str, TensorReq]:
        # a tied checkpoint may still carry the head; it is then ignored
        return {spec.name: TensorReq((spec.vocab_size, spec.hidden_size), optional=spec.tied)}

    def forward(self, h: torch.Tensor, step=None) -> torch.Tensor:
        # queued with the products before it; the model flushes the queue before it returns the logits
        logits = linear(h, self.weight, out_dtype=torch.float32, err=getattr(step, "err", None), chain=chain_of(step),
                        queue_plain=True)
        return sum_parts(logits, torch.float32)
