"""Replay of the same requests under every way of cutting them, against the plain implementation."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import tiny_configs
import traces
from helpers import model_folder, random_tokens

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"A": [5, 17, 33, 70, 130, 96, 41, 128], "B": [1, 7, 31, 64, 100, 143, 52, 90],
           "W": [3, 40, 77, 150, 64, 110, 25, 95], "C": [2, 19, 64, 129, 80, 47, 111, 96],
           "D": [4, 33, 65, 140, 90, 128, 31, 70], "O": [6, 50, 97, 130, 64, 33, 120, 80],
           "H": [3, 66, 120, 40, 90, 128, 17, 72]}
DTYPES = ["float32", "bfloat16"]


def requests_for(tag: str) -> dict:
    vocab = tiny_configs.ALL[tag][0]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS[tag])}


def make_core(tag: str, dtype: str, max_tokens: int):
    from tokamak_b200.engine.replay import build_core
    page = tiny_configs.ALL[tag][2]
    return build_core(model_folder(tag, dtype), dtype, max_tokens, page_size=page, max_live=4)


def replay(tag, dtype, builder, max_tokens, poison=False, **kw):
    from tokamak_b200.engine.replay import run_step
    reqs = requests_for(tag)
    if builder is traces.mixed:
        kw["max_tokens"] = max_tokens
    records, rows = builder(reqs, **kw)
    core = make_core(tag, dtype, max_tokens)
    results = {}
    for rec in records:
        if poison:
            core.cache.poison_free_pages()
        out = run_step(core, rec)
        if out is not None:
            results[rec["step"]] = out
        core.manager.check_invariants()
    assert not core.manager.live_requests()
    assert all(g.num_free == g.num_pages for g in core.manager.kv_groups)
    n = traces.check(results, rows, reqs, model_folder(tag, dtype), dtype, f"{tag}/{dtype}")
    assert n == sum(len(v) for v in rows.values())
    return core


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["A", "B", "W", "C", "D"])
def test_whole(tag, dtype):
    replay(tag, dtype, traces.whole, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["A", "B", "W", "C", "D"])
def test_tail_one_by_one(tag, dtype):
    replay(tag, dtype, traces.tail_one_by_one, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["A", "B", "W", "C", "D", "O", "H"])
def test_portions(tag, dtype):
    replay(tag, dtype, traces.portions, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["A", "B", "W", "C", "D", "O", "H"])
def test_mixed_with_page_reuse(tag, dtype):
    core = replay(tag, dtype, traces.mixed, max_tokens=384, poison=True, seed=7)
    # the pool is smaller than the sum of all requests, so pages were used again
    assert sum(LENGTHS[tag]) > 384


@pytest.mark.parametrize("seed", [1, 2, 3])
@pytest.mark.parametrize("tag,dtype", [("W", "float32"), ("D", "bfloat16"), ("C", "bfloat16"), ("B", "float32")])
def test_mixed_in_other_orders(tag, dtype, seed):
    """The mixed replay again with other random orders, portion sizes and pauses, and a smaller
    pool: windows that give pages back while other requests take them, poisoned free pages."""
    replay(tag, dtype, traces.mixed, max_tokens=320, poison=True, seed=seed)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decode(dtype):
    """Positions 0, 1, 2 one by one, then 220 more decoded one by one across many pages."""
    tag = "A"
    vocab = tiny_configs.ALL[tag][0]["vocab_size"]
    reqs = {"long": random_tokens(vocab, 224, seed=5)}
    records, rows = traces.tail_one_by_one(reqs, tail=223)
    from tokamak_b200.engine.replay import run_trace
    core = make_core(tag, dtype, 256)
    results = run_trace(core, records)
    traces.check(results, rows, reqs, model_folder(tag, dtype), dtype, f"long/{dtype}")


def test_same_logits_however_cut_float32():
    """In float32 the cuts agree with each other far more tightly than with the float64 truth."""
    from tokamak_b200.engine.replay import run_trace
    tag = "B"
    reqs = requests_for(tag)
    got = {}
    for name, builder in (("whole", traces.whole), ("portions", traces.portions)):
        records, rows = builder(reqs)
        res = run_trace(make_core(tag, "float32", 192), records)
        got[name] = {rp: res[s][i] for s in rows for i, rp in enumerate(rows[s])}
    for rp, a in got["whole"].items():
        b = got["portions"][rp]
        assert np.abs(a - b).max() <= 2e-5 * max(1.0, np.abs(a).max()), rp


def test_trace_run_program(tmp_path):
    """The command-line program end to end, on a short mixed trace in float32."""
    tag, dtype = "A", "float32"
    reqs = {k: v for k, v in list(requests_for(tag).items())[:4]}
    records, rows = traces.mixed(reqs, max_tokens=256, seed=3)
    folder = model_folder(tag, dtype)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
         "--out", str(out), "--max-tokens", "256"],
        input="".join(json.dumps(r) + "\n" for r in records), text=True, capture_output=True,
        timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for r in records for w in ("done", str(r["step"]))]
    vocab = tiny_configs.ALL[tag][0]["vocab_size"]
    results = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, vocab) for s in rows}
    traces.check(results, rows, reqs, folder, dtype, "trace_run")


def _random_config(seed: int) -> tuple[dict, int]:
    """A Qwen3 configuration drawn at random from what the configuration allows: head sizes in
    steps of 16, any number of heads and groups, widths and vocabularies that are no powers of two,
    one to three layers, with or without a window, tied or untied head."""
    import random
    rng = random.Random(seed)
    kv = rng.choice([1, 2, 3, 4])
    heads = kv * rng.choice([1, 2, 3, 5])
    cfg = {
        "architectures": ["Qwen3ForCausalLM"],
        "num_hidden_layers": rng.choice([1, 2, 3]),
        "hidden_size": 8 * rng.randrange(4, 30),
        "num_attention_heads": heads, "num_key_value_heads": kv,
        "head_dim": 16 * rng.randrange(1, 9),
        "intermediate_size": 8 * rng.randrange(5, 40),
        "vocab_size": rng.randrange(90, 400),
        "rope_theta": rng.choice([1e4, 5e4, 1e6]),
        "rms_norm_eps": rng.choice([1e-6, 1e-5]),
        "tie_word_embeddings": rng.random() < 0.5,
        "max_position_embeddings": 256,
    }
    if rng.random() < 0.4:
        cfg.update({"use_sliding_window": True, "sliding_window": rng.randrange(5, 60),
                    "max_window_layers": rng.randrange(0, cfg["num_hidden_layers"])})
    return cfg, rng.choice([8, 16, 32])


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Mixed replay with page reuse, in float32 and in bfloat16, for configurations drawn at random."""
    from tokamak_b200.engine.replay import build_core, run_step
    from tokamak_b200.weights import write_random_model
    cfg, page = _random_config(seed)
    lengths = [3, 47, 130, 64, 21, 90]
    reqs = {f"q{i}": random_tokens(cfg["vocab_size"], n, seed=31 * i + seed) for i, n in enumerate(lengths)}
    for dtype in DTYPES:
        folder = write_random_model(tmp_path / dtype, cfg, seed=seed, std=0.08, dtype=dtype)
        records, rows = traces.mixed(reqs, max_tokens=256, max_live=3, seed=seed)
        core = build_core(folder, dtype, 256, page_size=page, max_live=3)
        results = {}
        for rec in records:
            core.cache.poison_free_pages()
            out = run_step(core, rec)
            if out is not None:
                results[rec["step"]] = out
            core.manager.check_invariants()
        assert not core.manager.live_requests()
        traces.check(results, rows, reqs, folder, dtype, f"random configuration {seed} ({cfg}) in {dtype}")
