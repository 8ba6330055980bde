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


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_pages_beyond_four_gib_are_addressed_right(model_8b_sizes, dtype):
    """A pool whose per-layer key view alone is larger than 4 GiB, with every low page taken
    away first: the requests live in the last pages, more than 2^32 bytes and 2^31 elements into
    the view, and prefill, portions and decoding give the logits of the plain implementation."""
    from tokamak_b200.engine.core import EngineCore
    from tokamak_b200.engine.replay import run_step
    raw, tensors, cpu = model_8b_sizes
    elem = 2 if dtype == "bfloat16" else 4
    pool_tokens = 2_359_296 * 2 // elem           # 1024 key elements per token and layer: 4.5 GiB per view
    need = 4 * pool_tokens * 1024 * elem + (8 << 30)
    if torch.cuda.mem_get_info()[0] < need:
        pytest.skip("not enough free device memory for a pool beyond 4 GiB per view")
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    mine = {k: (v.float() if v.dim() == 1 else v.to(dt)) for k, v in tensors.items()}
    core = EngineCore("<random>", dtype=dtype, tensors=mine, raw_config=raw, max_seq_len=512,
                      page_size=16, pool_tokens=pool_tokens, max_slots=4, max_step_tokens=512)
    view = core.cache.view(next(iter(core.model.cache_needs())))
    assert view.k.numel() * view.k.element_size() > (1 << 32)
    assert dtype == "float32" or view.k.numel() > (1 << 31)
    for g in core.manager.kv_groups:
        g.allocator.take(g.num_free - 64)         # held by nobody's table: only the last 64 pages are left
    reqs = {"a": random_tokens(raw["vocab_size"], 300, seed=5), "b": random_tokens(raw["vocab_size"], 90, seed=6)}
    truth = {rid: plain.forward_logits(raw, cpu, ids, torch.float64) for rid, ids in reqs.items()}
    for builder, kw in ((traces.whole, {}), (traces.tail_one_by_one, {"tail": 8}),
                        (traces.mixed, {"max_tokens": 512, "max_live": 2, "seed": 3})):
        records, rows = builder(reqs, **kw)
        for rec in records:
            out = run_step(core, rec)
            if out is None:
                continue
            want = torch.stack([truth[rid][p] for rid, p in rows[rec["step"]]])
            assert_logits_close(torch.from_numpy(out), want, dtype, f"high pages {builder.__name__} {rec['step']}")
        assert not core.manager.live_requests()
    del core
    torch.cuda.empty_cache()


def test_a_long_prompt_through_the_products_for_many_tokens(model_8b_sizes):
    """A prompt of 1,024 tokens in one step: the projections with enough tiles run on pairs of SMs,
    the gate/up product with the activation in its epilogue; then eight tokens one by one."""
    from tokamak_b200.engine.core import EngineCore
    from tokamak_b200.engine.replay import run_step
    from tokamak_b200.csrc import ops
    raw, tensors, cpu = model_8b_sizes
    assert ops.pair_gemm_takes(1016, 2 * raw["intermediate_size"], raw["hidden_size"], fused=True)
    mine = {k: (v.float() if v.dim() == 1 else v) for k, v in tensors.items()}
    core = EngineCore("<random>", dtype="bfloat16", tensors=mine, raw_config=raw, max_seq_len=1024, page_size=16,
                      pool_tokens=1024, max_slots=2, max_step_tokens=1024)
    reqs = {"long": random_tokens(raw["vocab_size"], 1024, seed=9)}
    truth = plain.forward_logits(raw, cpu, reqs["long"], torch.float64)
    records, rows = traces.tail_one_by_one(reqs, tail=8)
    for rec in records:
        out = run_step(core, rec)
        want = torch.stack([truth[p] for _, p in rows[rec["step"]]])
        assert_logits_close(torch.from_numpy(out), want, "bfloat16", f"long prompt step {rec['step']}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", ["LAYER_14B", "LAYER_32B"])
def test_14b_and_32b_layer_sizes(sizes, dtype):
    """One layer of the widths, head counts and intermediate sizes of Qwen3-14B and Qwen3-32B (one
    layer keeps the float64 oracle on the CPU within seconds): a prompt whole with its tail token by
    token, and two requests mixed, one of them long enough for the products of many tokens."""
    from tokamak_b200.config import architecture_of
    from tokamak_b200.engine.replay import run_step
    from tokamak_b200.models.decoder import DecoderModel
    from tokamak_b200.weights import random_tensors
    raw = getattr(tiny_configs, sizes)
    arch = architecture_of(raw)
    expected = DecoderModel.expected_tensors(arch.model_spec(arch.parse_config(raw)))
    tensors = random_tensors(expected, seed=5, std=0.02, norm_std=0.1, dtype=torch.bfloat16, device="cuda")
    cpu = {k: v.float().cpu() for k, v in tensors.items()}
    reqs = {"a": random_tokens(raw["vocab_size"], 300, seed=3), "b": random_tokens(raw["vocab_size"], 45, seed=4)}
    truth = {rid: plain.forward_logits(raw, cpu, ids, torch.float64) for rid, ids in reqs.items()}
    del cpu
    core = make_core(raw, tensors, dtype)
    for builder, kw in ((traces.tail_one_by_one, {"tail": 6}), (traces.mixed, {"max_tokens": 512, "max_live": 2, "seed": 2})):
        records, rows = builder(reqs, **kw)
        for rec in records:
            out = run_step(core, rec)
            if out is None:
                continue
            want = torch.stack([truth[rid][p] for rid, p in rows[rec["step"]]])
            assert_logits_close(torch.from_numpy(out), want, dtype, f"{sizes} {builder.__name__} step {rec['step']}")
        assert not core.manager.live_requests()
