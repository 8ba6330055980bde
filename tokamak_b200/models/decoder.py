"""A decoder described as data: parts, blocks, and the order in which they run."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts import embedding as _builtin_embedding   # registers the built-in embedding and head
from ..parts.base import (BLOCKS, EMBEDDINGS, HEADS, NORMS, POSITIONS, OwedNorm, Runtime, TensorReq, graph_safe,
                          weight_bytes)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the schedule: which block runs and which cache it uses.

    Naming a block twice runs its weights twice; two calls that name the same
    ``cache`` share keys and values (the later one must be built without key and
    value projections of its own).  ``cache`` is ``None`` for a block that keeps
    nothing between steps.
    """

    block: str
    cache: str | None


@dataclass(frozen=True)
class ModelSpec:
    """A model as data.  Every field but the schedule is a spec with a ``kind`` that one of the
    registries of ``parts/base.py`` resolves; ``embedding_position`` is the seat of a position
    encoding that is added to the embedded rows (``None``: the mixers carry the positions)."""

    embedding: object                  # an embedding spec (vocab_size, hidden_size, kind, ...)
    blocks: tuple                      # block specs, each with a unique ``name``
    schedule: tuple                    # LayerCall entries, in execution order
    final_norm: object
    final_norm_name: str
    head: object                       # a head spec (vocab_size, kind, ...)
    embedding_position: object = None

    def __post_init__(self) -> None:
        names = [b.name for b in self.blocks]
        if len(set(names)) != len(names):
            raise ValueError("block names must be unique")
        for call in self.schedule:
            if call.block not in names:
                raise ValueError(f"the schedule names an unknown block {call.block!r}")


class DecoderModel:
    """Embedding, the scheduled blocks, final norm and head
    (src/tokamak/model/transformer.py:112-176), built from a :class:`ModelSpec`."""

    def __init__(self, spec: ModelSpec, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, tensors, rt)
        self.embedding_position = None
        if spec.embedding_position is not None:
            pos = spec.embedding_position
            self.embedding_position = POSITIONS.get(pos.kind)(pos, tensors, rt)
            if not hasattr(self.embedding_position, "add_to_embedding"):
                raise ValueError(f"position encoding {pos.kind!r} cannot sit at the embedding: "
                                 f"it has no add_to_embedding")
        self.blocks = {b.name: BLOCKS.get(b.kind)(b, tensors, rt) for b in spec.blocks}
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, spec.final_norm_name,
                                                          tensors, rt)
        self.head = HEADS.get(spec.head.kind)(spec.head, self.embedding, tensors, rt)

    @staticmethod
    def expected_tensors(spec: ModelSpec) -> dict[str, TensorReq]:
        out: dict[str, TensorReq] = {}
        out.update(EMBEDDINGS.get(spec.embedding.kind).expected_tensors(spec.embedding))
        if spec.embedding_position is not None:
            pos = spec.embedding_position
            out.update(POSITIONS.get(pos.kind).expected_tensors(pos))
        for b in spec.blocks:
            out.update(BLOCKS.get(b.kind).expected_tensors(b))
        out.update(NORMS.get(spec.final_norm.kind).expected_tensors(spec.final_norm,
                                                                    spec.final_norm_name))
        out.update(HEADS.get(spec.head.kind).expected_tensors(spec.head))
        return out

    def parts(self) -> list:
        """Every part a step runs, a block once per call of the schedule."""
        out = [self.embedding] + ([self.embedding_position] if self.embedding_position is not None else [])
        out += [self.blocks[call.block] for call in self.spec.schedule]
        return out + [self.final_norm, self.head]

    def graph_safe(self) -> bool:
        """Whether a step of single next tokens may be replayed from a CUDA graph: every part
        has to declare it (``GRAPH_SAFE`` in ``parts/base.py``)."""
        return graph_safe(*self.parts())

    def step_weight_bytes(self) -> int:
        """Bytes of weights that one step reads in full: every scheduled call's, the final norm's
        and the head's (what the parts report through ``weight_bytes``)."""
        return weight_bytes(*self.parts())

    def cache_needs(self) -> dict[str, object]:
        """Cache key -> need, checked for agreement between calls that share a key."""
        needs: dict[str, object] = {}
        for call in self.spec.schedule:
            need = self.blocks[call.block].cache_need()
            if need is None:
                if call.cache is not None:
                    raise ValueError(f"block {call.block!r} keeps no cache but is given {call.cache!r}")
                continue
            if call.cache is None:
                raise ValueError(f"block {call.block!r} needs a cache and the schedule names none")
            if call.cache in needs and needs[call.cache] != need:
                raise ValueError(f"cache {call.cache!r} is shared by blocks with different needs")
            needs.setdefault(call.cache, need)
        return needs

    def forward(self, step) -> torch.Tensor:
        """Float32 logits ``[len(step.logits_rows), vocab]`` for the rows asked for."""
        resid = self.embedding.forward(step)
        if self.embedding_position is not None:
            self.embedding_position.add_to_embedding(resid, step)
        pending = None
        schedule = self.spec.schedule
        for i, call in enumerate(schedule):
            view = step.cache.view(call.cache) if call.cache is not None else None
            block = self.blocks[call.block]
            if getattr(block, "TAKES_NEXT_NORM", False):
                # the norm that will consume what the block leaves pending: the next block's, or the last
                after = self.blocks[schedule[i + 1].block] if i + 1 < len(schedule) else None
                next_norm = getattr(after, "entry_norm", None) if after is not None else self.final_norm
                resid, pending = block.forward(resid, pending, step, view, next_norm=next_norm)
            else:
                resid, pending = block.forward(resid, pending, step, view)
        if step.n_want == 0:
            return torch.empty((0, self.spec.head.vocab_size), dtype=torch.float32, device=resid.device)
        # every request brings one token and wants it: the wanted rows are all rows, in order
        all_rows = step.n_want == step.n_tokens and step.max_q_len == 1
        h = self.final_norm.add_norm(resid, pending, rows=None if all_rows and isinstance(pending, OwedNorm) else step.logits_rows)
        if isinstance(h, OwedNorm) and not getattr(self.head, "TAKES_OWED_NORM", False):
            h = h.materialize()
        logits = self.head.forward(h, step)
        from ..csrc import ops
        ops.flush_chains()          # products that are still queued: the caller reads the logits
        return logits
