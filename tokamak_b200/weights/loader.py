"""Reads safetensors by tensor name and checks the folder against what the model expects.

The reference binds by exact name and fails on the first problem
(src/tokamak/model/loader.py:54-95).  Here every problem of a folder is
collected and raised as one error that lists the missing tensors, the unexpected
ones and the wrong shapes.
"""

from __future__ import annotations

from pathlib import Path
from typing import Mapping

import torch

from ..parts.base import TensorReq


class WeightsError(ValueError):
    """The checkpoint does not match the model.

    Attributes ``missing``, ``unexpected`` and ``wrong_shape`` hold the lists.
    """

    def __init__(self, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple, tuple]], folder: str):
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        lines = [f"checkpoint under {folder} does not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} checkpoint {tuple(c)} vs model {tuple(m)}" for n, c, m in wrong_shape))
        super().__init__("\n".join(lines))


def checkpoint_files(model_dir: str | Path) -> list[Path]:
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"No *.safetensors files found under {model_dir}")
    return files


def target_dtype(req: TensorReq, stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    """Element type in memory: matrices follow the engine, per-channel vectors are
    float32 (exact for bfloat16 and for 32-bit storage), integer tables are int32."""
    if req.role == "int_table" or not stored.is_floating_point:
        return torch.int32
    if req.role == "vector":
        return torch.float32
    return engine_dtype


def load_tensors(model_dir: str | Path, expected: Mapping[str, TensorReq], engine_dtype: torch.dtype,
                 device: torch.device | str) -> dict[str, torch.Tensor]:
    """Every expected tensor, on ``device``, or one :class:`WeightsError` naming all faults."""
    from safetensors import safe_open

    files = checkpoint_files(model_dir)
    # first pass: names and shapes only, so that a faulty folder fails before any copy
    where: dict[str, Path] = {}
    unexpected: list[str] = []
    wrong: list[tuple[str, tuple, tuple]] = []
    for file in files:
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                if name not in expected:
                    unexpected.append(name)
                    continue
                shape = tuple(f.get_slice(name).get_shape())
                if shape != tuple(expected[name].shape):
                    wrong.append((name, shape, tuple(expected[name].shape)))
                where[name] = file
    missing = [n for n, req in expected.items() if n not in where and not req.optional]
    if missing or unexpected or wrong:
        raise WeightsError(sorted(missing), sorted(unexpected), sorted(wrong), str(model_dir))

    out: dict[str, torch.Tensor] = {}
    for file in files:
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                out[name] = t.to(device=device, dtype=target_dtype(expected[name], t.dtype, engine_dtype))
    return out
