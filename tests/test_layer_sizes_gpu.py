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
    expected = DecoderModel.expected_tensors(arch.build_spec(arch.parse(raw)))
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
    expected = DecoderModel.expected_tensors(arch.build_spec(arch.parse(raw)))
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


# ----------------------------------------------------------------------------- the serving path

def _margin_check(raw, cpu, prompt, generated, what):
    """Every generated token lies within a small margin of the plain maximum for its own prefix
    (bfloat16 may flip a near-tie; after that the prefix is the engine's, so the check goes on)."""
    seq = list(prompt) + list(generated)
    logits = plain.forward_logits(raw, cpu, seq[:-1], torch.float64)
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        gap = float(row.max() - row[tok])
        assert gap <= 0.04 * float(row.std()), f"{what}: token {i} is {gap:.4f} below the plain maximum"


@pytest.mark.parametrize("batch", [8, 64])
def test_generate_at_8b_sizes_with_graphs_and_steps_launched_ahead(model_8b_sizes, batch):
    """The path that serving and the benchmark take: bfloat16 at the Qwen3-8B layer sizes (the
    owed norms need a width that is a multiple of 128, the q|k|v epilogue heads of 128), decode
    steps driven by the slot records, replayed from CUDA graphs and launched one ahead.  Every
    token must be (nearly) the plain implementation's best for its prefix, and all tokens must
    equal those of the same engine with every step laid out by the host, one at a time, no graph."""
    from tokamak_b200 import LLM, SamplingParams
    from tokamak_b200.engine.core import EngineCore
    raw, tensors, cpu = model_8b_sizes
    mine = {k: (v.float() if v.dim() == 1 else v) for k, v in tensors.items()}
    core = EngineCore("<random>", dtype="bfloat16", tensors=mine, raw_config=raw, max_seq_len=256, page_size=16,
                      pool_tokens=batch * 256, max_slots=batch, max_step_tokens=1024)
    llm = LLM("<random>", _core=core, max_batch_size=batch, max_num_batched_tokens=1024, block_size=16)
    prompts = [random_tokens(raw["vocab_size"], 9 + (5 * i) % 23, seed=40 + i) for i in range(batch)]
    params = SamplingParams(temperature=0.0, max_new_tokens=44, ignore_eos=True)
    fast = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert core.step.graph_replays >= 30 and llm.last_stats["decode_steps"] >= 40
    llm.plain_steps = True
    replays = core.step.graph_replays
    slow = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert core.step.graph_replays == replays
    assert [o.output_token_ids for o in fast] == [o.output_token_ids for o in slow]
    for i in range(0, batch, max(1, batch // 6)):
        _margin_check(raw, cpu, prompts[i], fast[i].output_token_ids, f"batch {batch} request {i}")


def test_state_driven_steps_at_8b_sizes_equal_host_laid_steps(model_8b_sizes):
    """launch_and_sample from the slot records (graphs, two steps in flight, seeded temperature
    sampling) against run_and_sample with host tokens and host counters, at the 8B layer sizes."""
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    raw, tensors, _ = model_8b_sizes
    core = make_core(raw, tensors, "bfloat16")
    step = core.step
    prompts = [random_tokens(raw["vocab_size"], n, seed=n) for n in (33, 5, 17, 64)]
    rows = lambda k: [SamplingRow(0.8, 50, 0.95, seed=7 + i, counter=k) for i in range(4)]
    steps = 10

    def by_host(ids):
        toks = step.run_and_sample([StepEntry(r, p, [len(p) - 1]) for r, p in zip(ids, prompts)], rows(0))
        out = [toks]
        for k in range(1, steps):
            toks = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)], rows(k))
            out.append(toks)
        for r in ids:
            step.free(r)
        return out

    def by_device(ids):
        for r, row in zip(ids, rows(0)):
            step.admit(r, row)
        flight = step.launch_and_sample([StepEntry(r, p, [len(p) - 1]) for r, p in zip(ids, prompts)])
        out = []
        for _ in range(1, steps):
            ahead = step.launch_and_sample([StepEntry(r, None, [0]) for r in ids])
            out.append(step.collect(flight))
            flight = ahead
        out.append(step.collect(flight))
        for r in ids:
            step.free(r)
        return out

    want = by_host(["h0", "h1", "h2", "h3"])
    assert by_device(["d0", "d1", "d2", "d3"]) == want
    replays = step.graph_replays
    assert by_device(["e0", "e1", "e2", "e3"]) == want
    assert step.graph_replays >= replays + steps - 2


def test_one_layer_with_the_real_vocabulary():
    """The head of 151,936 rows (1,187 row tiles of the decode product, the library branch for
    more than 64 rows of float32 logits) inside a model: one layer of the 8B sizes, a prompt whole
    (every position wanted) and its last tokens one by one, against the plain implementation."""
    from tokamak_b200.config import architecture_of
    from tokamak_b200.engine.core import EngineCore
    from tokamak_b200.engine.replay import run_step
    from tokamak_b200.models.decoder import DecoderModel
    from tokamak_b200.weights import random_tensors
    raw = dict(tiny_configs.LAYER_8B, num_hidden_layers=1, vocab_size=151936, max_position_embeddings=256)
    arch = architecture_of(raw)
    expected = DecoderModel.expected_tensors(arch.build_spec(arch.parse(raw)))
    tensors = random_tensors(expected, seed=3, std=0.02, norm_std=0.1, dtype=torch.bfloat16, device="cuda")
    cpu = {k: v.float().cpu() for k, v in tensors.items()}
    mine = {k: (v.float() if v.dim() == 1 else v) for k, v in tensors.items()}
    core = EngineCore("<random>", dtype="bfloat16", tensors=mine, raw_config=raw, max_seq_len=256, page_size=16,
                      pool_tokens=256, max_slots=2, max_step_tokens=256)
    reqs = {"v": random_tokens(raw["vocab_size"], 80, seed=12)}
    truth = plain.forward_logits(raw, cpu, reqs["v"], torch.float64)
    for builder, kw in ((traces.whole, {}), (traces.tail_one_by_one, {"tail": 6})):
        records, rows = builder(reqs, **kw)
        for rec in records:
            out = run_step(core, rec)
            want = torch.stack([truth[p] for _, p in rows[rec["step"]]])
            assert_logits_close(torch.from_numpy(out), want, "bfloat16", f"real vocabulary {builder.__name__}")
