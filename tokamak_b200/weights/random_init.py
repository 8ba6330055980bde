"""Seeded random weights: a model folder from a configuration and a seed.

Matrices and the embedding are drawn from N(0, std), norm weights from
1 + N(0, norm_std), tensor after tensor in the order of the model's expected
names from one CPU generator, so that a (configuration, seed) pair names one
model.  The folder holds ``config.json`` and ``model.safetensors`` under the
checkpoint names, so anything that reads such folders can load it.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch

from ..config.registry import architecture_of
from ..parts.base import TensorReq

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(expected: Mapping[str, TensorReq], seed: int, std: float = 0.02,
                   norm_std: float = 0.1, dtype: torch.dtype = torch.bfloat16,
                   device: str | torch.device = "cpu") -> dict[str, torch.Tensor]:
    """One random tensor per expected name (optional ones are left out)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name, req in expected.items():
        if req.optional:
            continue
        if req.role == "vector":
            t = 1.0 + norm_std * torch.randn(req.shape, generator=gen, dtype=torch.float32, device=device)
        elif req.role == "int_table":
            t = torch.zeros(req.shape, dtype=torch.int32, device=device)
        else:
            t = std * torch.randn(req.shape, generator=gen, dtype=torch.float32, device=device)
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return out


def write_random_model(folder: str | Path, config_json: Mapping, seed: int, std: float = 0.02,
                       norm_std: float = 0.1, dtype: str | torch.dtype = "bfloat16") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a raw configuration dictionary."""
    from safetensors.torch import save_file

    from ..models.decoder import DecoderModel

    if isinstance(dtype, str):
        dtype = _DTYPES[dtype]
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = architecture_of(config_json)
    expected = DecoderModel.expected_tensors(arch.build_spec(arch.parse(config_json)))
    tensors = random_tensors(expected, seed, std, norm_std, dtype)
    raw = dict(config_json)
    raw.setdefault("torch_dtype", "bfloat16" if dtype == torch.bfloat16 else "float32")
    (folder / "config.json").write_text(json.dumps(raw, indent=2))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
