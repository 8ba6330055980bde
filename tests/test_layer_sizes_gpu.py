"""The engine at the layer sizes of Qwen3-8B (two layers, small vocabulary): float32 and bfloat16
against the plain implementation, whole, in portions and token by token."""

from __future__ import annotations

import pytest
import torch

import tiny_configs
import traces
from helpers import assert_logits_close, random_tokens
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_8b_sizes():
    """Seeded random weights made on the device, rounded to bfloat16 so that both engine dtypes
    and the plain implementation see the same values."""
    from tokamak_b200.config import architecture_of
    from tokamak_b200.models.decoder import DecoderModel
    from tokamak_b200.weights import random_tensors
    raw = tiny_configs.LAYER_8B
    arch = architecture_of(raw)
    expected = DecoderModel.expected_tensors(arch.model_spec(arch.parse_config(raw)))
    tensors = random_tensors(expected, seed=11, std=0.02, norm_std=0.1, dtype=torch.bfloat16, device="cuda")
    cpu = {k: v.float().cpu() for k, v in tensors.items()}
    return raw, tensors, cpu


def make_core(raw, tensors, dtype):
    from tokamak_b200.engine.core import EngineCore
    from tokamak_b200.parts.base import TensorReq
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    mine = {k: (v.float() if v.dim() == 1 else v.to(dt)) for k, v in tensors.items()}
    return EngineCore("<random>", dtype=dtype, tensors=mine, raw_config=raw, max_seq_len=512, page_size=16,
                      pool_tokens=1024, max_slots=4, max_step_tokens=512)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_8b_layer_sizes_under_every_cut(model_8b_sizes, dtype):
    from tokamak_b200.engine.replay import run_step
    raw, tensors, cpu = model_8b_sizes
    reqs = {"a": random_tokens(raw["vocab_size"], 150, seed=1), "b": random_tokens(raw["vocab_size"], 70, seed=2)}
    truth = {rid: plain.forward_logits(raw, cpu, ids, torch.float64) for rid, ids in reqs.items()}
    core = make_core(raw, tensors, dtype)
    for builder, kw in ((traces.whole, {}), (traces.tail_one_by_one, {"tail": 12}),
                        (traces.portions, {"sizes": (40, 2, 64, 1, 17)}),
                        (traces.mixed, {"max_tokens": 512, "max_live": 2, "seed": 1})):
        records, rows = builder(reqs, **kw)
        for rec in records:
            # keep the comparison light: check only the last wanted row of every entry
            out = run_step(core, rec)
            got = torch.from_numpy(out)
            want = torch.stack([truth[rid][p] for rid, p in rows[rec["step"]]])
            assert_logits_close(got, want, dtype, f"8B sizes {builder.__name__} step {rec['step']}")
        assert not core.manager.live_requests()
