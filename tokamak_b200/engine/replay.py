"""Trace replay over the engine's own step function, cache and kernels.

A trace is a list of steps; a step names, for some requests, their next tokens
and the places among them whose logits are wanted, and the requests that end
after it.  Nothing is sampled.  ``bin/trace_run`` is the command-line form.
"""

from __future__ import annotations

import os
from pathlib import Path
from typing import Callable, Iterable

import numpy as np
import torch

from ..config import read_config_json
from .core import EngineCore
from .step import StepEntry


def build_core(model: str | Path, dtype: str, max_tokens: int, page_size: int = 16,
               max_live: int = 8) -> EngineCore:
    """An engine whose page pool holds ``max_tokens`` positions, rounded up to whole pages."""
    if page_size < 1 or 64 % page_size:
        raise ValueError("the page size must divide 64")
    pool_tokens = -(-max_tokens // page_size) * page_size
    model_max = int(read_config_json(model).get("max_position_embeddings", pool_tokens))
    return EngineCore(model, dtype=dtype, max_seq_len=min(model_max, pool_tokens),
                      page_size=page_size, pool_tokens=pool_tokens, max_slots=max_live,
                      max_step_tokens=pool_tokens)


def run_step(core: EngineCore, record: dict) -> np.ndarray | None:
    """Run one step record; float32 logits [wanted, vocab] or ``None`` if nothing was wanted."""
    entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in record.get("entries", [])]
    out = None
    if entries:
        logits = core.step.run(entries)
        if logits.shape[0] > 0:
            out = logits.to("cpu", torch.float32).contiguous().numpy()
    for req_id in record.get("end", []):
        core.step.free(req_id)
    return out


def run_trace(core: EngineCore, records: Iterable[dict], out_dir: str | Path | None = None,
              report: Callable[[object], None] | None = None) -> dict:
    """Replay the records in order; returns ``{step: logits}`` and writes ``<step>.f32`` files."""
    results: dict = {}
    if out_dir is not None:
        out_dir = Path(out_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
    for record in records:
        step_no = record["step"]
        arr = run_step(core, record)
        if arr is not None:
            results[step_no] = arr
            if out_dir is not None:
                tmp = out_dir / f".{step_no}.f32.tmp"
                arr.astype("<f4", copy=False).tofile(tmp)
                os.replace(tmp, out_dir / f"{step_no}.f32")
        if report is not None:
            report(step_no)
    return results
