"""Headline measurement: decode tokens per second of the Qwen3-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A *step* is one decode step: every live request advances by one token (model
forward over the paged cache, greedy sampling on the device, one copy of the
tokens back).  The default run has the layer sizes of Qwen3-8B with seeded
random bfloat16 weights, a batch of 8 and a context that ends at 4,096 tokens.
It prints ONE JSON line:

  value      decoded tokens per second at the default batch, timed with CUDA events
  e2e        the same through ``LLM.generate`` (host token ids in, host token ids out)
  prefill    one 2,048-token prompt in one step: tokens/s, ms, fraction of the bf16 peak
  roofline   bytes the decode step must read (weights once + live cache) / its time
  points     decode tokens per second at batch 1 and 64
  clocks     SM clocks and throttle reasons sampled during the timed regions

The engine runs on one GPU only: for ``--gpus N`` with N > 1 it says so and exits with 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960,
}
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40,
                 intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 intermediate_size=25600)
SIZES = {"8b": ("Qwen3-8B", QWEN3_8B), "14b": ("Qwen3-14B", QWEN3_14B), "32b": ("Qwen3-32B", QWEN3_32B)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PROMPT_PORTION = PREFILL_TOKENS
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi in the background, sampling clocks and throttle reasons (reading only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.file = None

    def start(self) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def bench_config(model_name: str, raw: dict, layers_of_model: int, batch: int, ctx: int, pf_tokens: int,
                 peaks_source: str) -> dict:
    """The ``config`` record of the bench line: every size, flat.  Both arms (this engine and the
    reference) print the same record for the same run."""
    return {
        "model": f"{model_name} layer sizes", "layers": raw["num_hidden_layers"], "layers_of_model": layers_of_model,
        "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"],
        "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
        "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "rope_theta": raw["rope_theta"],
        "rms_norm_eps": raw["rms_norm_eps"], "tied_head": bool(raw.get("tie_word_embeddings", False)),
        "global_batch": batch, "seq_len": ctx, "prefill_tokens": pf_tokens, "kv_block": 16,
        "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read every step)",
        "peaks": peaks_source,
    }


def weight_bytes(core) -> int:
    """Bytes of every weight a decode step reads once, as the model's parts report them (the
    embedding table is read by row only and reports nothing)."""
    return core.model.step_weight_bytes()


def step_flops(cfg, n_layers: int, tokens: int, ctx_start: int = 0) -> float:
    """Multiply-adds of a step of ``tokens`` new tokens of one request, counted as 2 flops."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    hq, hkv, inter = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"]
    per_layer = 2.0 * tokens * (h * (hq + 2 * hkv) * d + hq * d * h + 3 * h * inter)
    # causal attention: token i sees ctx_start + i + 1 keys; QK^T and PV
    keys = tokens * ctx_start + tokens * (tokens + 1) / 2
    per_layer += 2.0 * 2.0 * keys * hq * d
    return n_layers * per_layer + 2.0 * 1 * h * cfg["vocab_size"]


def fill_context(core, req_ids, length: int, vocab: int, seed: int) -> None:
    """Put ``length`` random tokens of every request into the cache, in prompts and prompt
    portions of ``PROMPT_PORTION`` tokens a step (2,048 unless ``--prompt-tokens`` says otherwise)."""
    import torch
    from tokamak_b200.engine.step import StepEntry
    gen = torch.Generator().manual_seed(seed)
    for rid in req_ids:
        toks = torch.randint(0, vocab, (length,), generator=gen).tolist()
        for s in range(0, length, PROMPT_PORTION):
            core.step.run([StepEntry(rid, toks[s:s + PROMPT_PORTION], [])], check=False)
    core.step.check_errors()


def time_decode(core, batch: int, steps: int, warmup: int, ctx_end: int, vocab: int, sampling=None):
    """Device time of ``steps`` decode steps of ``batch`` requests whose context ends at ``ctx_end``.

    The steps run as generation runs them: each request's token, position and sampling state
    are in its slot record on the device, the step is replayed from a CUDA graph, and it is
    launched one ahead, before the host has read the step before it; every step's tokens still
    come back to the host.  Afterwards the same requests are rewound and the same steps run
    again kernel by kernel, without graphs and without launching ahead: the tokens must be the
    same, or the timed path computed something else than the plain path."""
    import torch
    from tokamak_b200.csrc import ops
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    step = core.step
    req_ids = [f"b{batch}_{i}" for i in range(batch)]
    start_len = ctx_end - (steps + warmup + 1)
    for rid in req_ids:
        # greedy, or (temperature, top_k, top_p) with a seed per request
        step.admit(rid, SamplingRow() if sampling is None else
                   SamplingRow(temperature=sampling[0], top_k=int(sampling[1]), top_p=sampling[2], seed=1 + len(rid)))
    fill_context(core, req_ids, start_len - 1, vocab, seed=batch)
    last = [1 + i for i in range(batch)]
    # the last prompt token of every request, sampled: from here on the records carry the requests
    first = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(req_ids, last)])
    entries = [StepEntry(r, None, [0]) for r in req_ids]
    produced = [first]

    flight = step.launch_and_sample(entries)

    def one_step():
        nonlocal flight
        ahead = step.launch_and_sample(entries)
        produced.append(step.collect(flight))
        flight = ahead

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    launches0 = ops.LAUNCHES + step.graph_launches
    h2d0, d2h0 = step.buffers.h2d_bytes, step.buffers.d2h_bytes
    t_host = time.perf_counter()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    produced.append(step.collect(flight))
    ms = begin.elapsed_time(end)
    wall = time.perf_counter() - t_host
    launches = ops.LAUNCHES + step.graph_launches - launches0
    h2d, d2h = step.buffers.h2d_bytes - h2d0, step.buffers.d2h_bytes - d2h0
    kv_bytes = batch * (ctx_end - steps / 2.0) * core.cache.bytes_per_token()

    # the check: rewind every request to where the records took over and decode again, plainly
    replays = step.graph_replays
    for rid in req_ids:
        if sampling is None:
            step.restart(rid)
        else:           # a restarted request keeps its generator's count, as after a preemption: begin anew instead
            step.free(rid)
            step.admit(rid, SamplingRow(temperature=sampling[0], top_k=int(sampling[1]), top_p=sampling[2],
                                        seed=1 + len(rid)))
    fill_context(core, req_ids, start_len - 1, vocab, seed=batch)
    graphs, step.use_graphs = step.use_graphs, False
    toks = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(req_ids, last)])
    checked = toks == produced[0]
    for want in produced[1:]:
        toks = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(req_ids, toks)])
        checked = checked and toks == want
    step.use_graphs = graphs
    assert step.graph_replays == replays
    for r in req_ids:
        step.free(r)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "kv_bytes": kv_bytes, "wall_ms_per_step": wall * 1e3 / steps, "checked": checked,
            "graph_replays": replays, "h2d_bytes_per_step": h2d / steps, "d2h_bytes_per_step": d2h / steps}


def time_prefill(core, vocab: int, tokens: int = PREFILL_TOKENS, repeats: int = 3):
    import torch
    from tokamak_b200.engine.step import StepEntry
    gen = torch.Generator().manual_seed(99)
    times = []
    for i in range(repeats + 1):
        toks = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
        rid = f"prefill{i}"
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        core.step.run([StepEntry(rid, toks, [tokens - 1])], check=False)
        end.record()
        torch.cuda.synchronize()
        core.step.free(rid)
        if i > 0:
            times.append(begin.elapsed_time(end))
    core.step.check_errors()
    return statistics.median(times)


def time_e2e(core, batch: int, steps: int, warmup: int, ctx_end: int, vocab: int):
    """Decode tokens per second through ``LLM.generate``: host token ids in and out."""
    import torch
    from tokamak_b200 import LLM, SamplingParams
    # a budget that takes every prompt in one step, so that all requests decode together
    llm = LLM("<random>", _core=core, max_batch_size=batch, max_num_batched_tokens=batch * ctx_end,
              block_size=core.page_size)
    gen = torch.Generator().manual_seed(7)
    # the prompts of all requests are prefilled in one burst under the power cap, and the first
    # two dozen decode steps after it run at clocks that are still recovering (5.4, 4.7, 4.2 ms,
    # then 3.8 ms per step at batch 8): they count as warm-up here
    warmup = max(warmup, 32)
    new_tokens = steps + warmup + 1
    prompt_len = ctx_end - new_tokens
    prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).tolist() for _ in range(batch)]
    params = SamplingParams(temperature=0.0, max_new_tokens=new_tokens, ignore_eos=True)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert all(len(o.output_token_ids) == new_tokens for o in outs)
    times = llm.last_stats["decode_step_times"]
    assert len(times) >= steps + warmup, "the requests did not decode together"
    full = times[-steps:]                         # the last K decode steps, all at full batch
    tok_s = batch * len(full) / sum(full)
    # bytes copied to the device in those steps, counted from the copies the step function made: a
    # decode step's description lives in the slot records on the device, so what is copied is the
    # block-table entries of new pages (a new page every 16 tokens of a request) and, when the set
    # of running requests changes, the list of their slots
    h2d = sum(llm.last_stats["decode_step_h2d_bytes"][-steps:]) / len(full)
    d2h = 4 * (4 + batch)
    return {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": round(h2d, 1), "d2h_bytes_per_step": d2h,
            "ms_per_step": 1e3 * sum(full) / len(full), "warmup_steps": warmup}


QWEN3_0_6B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960,
}


def throughput_requests(num_requests: int, max_new_cap: int, seed: int, vocab: int):
    """The requests of the reference's throughput benchmark (benchmarks/workload.py:23-48): prompt
    lengths log-normal(5.0, 0.7) clipped to 16..512, new tokens 8 + exponential(mean 120) capped,
    random token ids folded below the first special token.  The draws are made in the
    reference's order, so that the default arguments give its 4,915 prompt and 2,901 output tokens."""
    import random
    rng = random.Random(seed)
    prompts, new_tokens = [], []
    for _ in range(num_requests):
        length = int(min(max(rng.lognormvariate(5.0, 0.7), 16), 512))
        new_tokens.append(min(int(rng.expovariate(1 / 120)) + 8, max_new_cap))
        prompts.append([rng.randrange(vocab) % 151_643 for _ in range(length)])
    return prompts, new_tokens


def throughput_workload(sizes: str, num_requests: int, max_new_cap: int, batch: int, pool_tokens: int,
                        seed: int) -> dict:
    """Output tokens per second of ``LLM.generate`` over the reference's 32-request workload
    (benchmarks/benchmark_throughput.py:31-68: continuous batching, EOS ignored, greedy)."""
    import torch
    from tokamak_b200 import LLM, SamplingParams
    from tokamak_b200.engine.core import random_core
    raw = dict(QWEN3_0_6B if sizes == "0.6b" else QWEN3_8B)
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=1024, page_size=16,
                       pool_tokens=pool_tokens, max_slots=batch, max_step_tokens=2048)
    llm = LLM("<random>", _core=core, max_batch_size=batch, max_num_batched_tokens=2048, block_size=16)
    prompts, new_tokens = throughput_requests(num_requests, max_new_cap, seed, raw["vocab_size"])
    params = [SamplingParams(temperature=0.0, max_new_tokens=n, ignore_eos=True) for n in new_tokens]
    llm.generate(prompt_token_ids=prompts, sampling_params=params)          # warm-up: graphs, allocator
    runs = []                  # the median of three runs, as the reference reports (benchmarks/README.md:3-5)
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
        torch.cuda.synchronize()
        runs.append((time.perf_counter() - t0, outs, dict(llm.last_stats)))
    runs.sort(key=lambda r: r[0])
    wall, outs, stats = runs[1]
    n_out = sum(len(o.output_token_ids) for o in outs)
    ttft = sorted(o.ttft_s for o in outs)
    lat = sorted(o.latency_s for o in outs)
    return {"workload": "throughput (reference's 32 seeded requests)", "sizes": f"Qwen3-{sizes.upper()} layer sizes",
            "requests": num_requests, "prompt_tokens": sum(len(p) for p in prompts), "output_tokens": n_out,
            "max_batch_size": batch, "kv_pool_tokens": pool_tokens, "output_tok_s": round(n_out / wall, 1),
            "wall_s": round(wall, 3), "wall_s_runs": [round(r[0], 3) for r in runs], "ttft_mean_s": round(sum(ttft) / len(ttft), 4),
            "ttft_p99_s": round(ttft[-1], 4), "latency_mean_s": round(sum(lat) / len(lat), 4),
            "steps": stats["steps"], "mixed_steps": stats["mixed_steps"],
            "preemptions": stats["preemptions"], "dtype": "bf16", "data": "synthetic"}


def mixed_workload(sizes: str, num_requests: int, new_tokens: int, chunk: int, seed: int) -> dict:
    """A mixed batch through ``LLM.generate``: ``num_requests`` requests with prompt lengths uniform
    in 128..4,096, all submitted at once, prompts computed in portions of ``chunk`` tokens beside the
    decode tokens of the requests that already run, ``new_tokens`` greedy tokens each, context limit
    8,192.  Every request runs from the start (a pool for all of them), so all but the first steps
    are mixed steps until the last prompt is done."""
    import random
    import torch
    from tokamak_b200 import LLM, SamplingParams
    from tokamak_b200.engine.core import random_core
    raw = dict(QWEN3_0_6B if sizes == "0.6b" else SIZES[sizes][1])
    rng = random.Random(seed)
    lengths = [rng.randint(128, 4096) for _ in range(num_requests)]
    prompts = [[rng.randrange(raw["vocab_size"]) for _ in range(n)] for n in lengths]
    pool = sum(-(-(n + new_tokens) // 16) * 16 for n in lengths)
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=8192, page_size=16,
                       pool_tokens=max(pool, 8192), max_slots=num_requests,
                       max_step_tokens=chunk + num_requests)
    llm = LLM("<random>", _core=core, max_batch_size=num_requests, max_num_batched_tokens=chunk + num_requests,
              prefill_chunk=chunk, block_size=16)
    params = SamplingParams(temperature=0.0, max_new_tokens=new_tokens, ignore_eos=True)
    llm.generate(prompt_token_ids=prompts, sampling_params=params)          # warm-up
    runs = []
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
        torch.cuda.synchronize()
        runs.append((time.perf_counter() - t0, outs, dict(llm.last_stats)))
    runs.sort(key=lambda r: r[0])
    wall, outs, stats = runs[1]
    n_out = sum(len(o.output_token_ids) for o in outs)
    ttft = sorted(o.ttft_s for o in outs)
    return {"workload": "mixed batch (prompt portions beside decode tokens)", "sizes": f"Qwen3-{sizes.upper()} layer sizes",
            "requests": num_requests, "prompt_tokens": sum(lengths), "output_tokens": n_out,
            "prefill_chunk": chunk, "max_seq_len": 8192, "kv_pool_tokens": max(pool, 8192),
            "total_tok_s": round((sum(lengths) + n_out) / wall, 1), "output_tok_s": round(n_out / wall, 1),
            "wall_s": round(wall, 3), "wall_s_runs": [round(r[0], 3) for r in runs],
            "ttft_mean_s": round(sum(ttft) / len(ttft), 4), "ttft_max_s": round(ttft[-1], 4),
            "steps": stats["steps"], "mixed_steps": stats["mixed_steps"], "preemptions": stats["preemptions"],
            "dtype": "bf16", "data": "synthetic"}


def latency_workload(sizes: str, prompt_tokens: int, new_tokens: int, iters: int, seed: int) -> dict:
    """Single-sequence latency as the reference measures it (benchmarks/benchmark_latency.py:63-97,
    119-133): one seeded random prompt, time to the first token (prefill, argmax on the host side
    of a sync), then greedy steps one by one with the token read back every step; medians of
    ``iters`` runs after a warm-up."""
    import torch
    from tokamak_b200.engine.core import random_core
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    raw = dict(QWEN3_0_6B if sizes == "0.6b" else SIZES[sizes][1])
    total = prompt_tokens + new_tokens
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=total, page_size=16,
                       pool_tokens=2 * total, max_slots=2, max_step_tokens=max(prompt_tokens, 64))
    gen = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, raw["vocab_size"], (prompt_tokens,), generator=gen).tolist()

    def run_once(i: int) -> tuple[float, float]:
        rid = f"lat{i}"
        core.step.admit(rid, SamplingRow())
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        token = core.step.run_and_sample([StepEntry(rid, prompt, [prompt_tokens - 1])])[0]
        t1 = time.perf_counter()
        for _ in range(new_tokens):
            token = core.step.run_and_sample([StepEntry(rid, None, [0])])[0]
        t2 = time.perf_counter()
        core.step.free(rid)
        return (t1 - t0) * 1e3, new_tokens / (t2 - t1)

    run_once(-1)
    runs = [run_once(i) for i in range(iters)]
    prefill_ms = statistics.median(r[0] for r in runs)
    tok_s = statistics.median(r[1] for r in runs)
    return {"workload": "latency (reference's single-sequence measurement)", "sizes": f"Qwen3-{sizes.upper()} layer sizes",
            "prompt_tokens": prompt_tokens, "new_tokens": new_tokens, "prefill_ms": round(prefill_ms, 3),
            "prefill_tok_s": round(prompt_tokens / (prefill_ms / 1e3), 1), "decode_tok_s": round(tok_s, 1),
            "inter_token_ms": round(1e3 / tok_s, 3), "iters": iters, "dtype": "bf16", "data": "synthetic"}


def kernel_case(name: str, batch: int, ctx: int, iters: int, peaks: dict, portion: int = 0, sizes: str = "8b",
                sampling=None) -> dict:
    """One kernel alone on inputs larger than L2, timed with CUDA events: achieved bytes or flops
    per second against the peak.  Also the small case that ncu captures are made on."""
    import torch
    from tokamak_b200.csrc import ops
    dev = "cuda"
    cfg = SIZES[sizes][1] if sizes in SIZES else QWEN3_8B
    hq, hkv, d, page = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], 16
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    flops = 0.0
    if name in ("attention_decode", "attention_decode_split", "attention_prefill", "attention_prefill_mma"):
        pages_per_req = -(-ctx // page)
        num_pages = batch * pages_per_req
        kc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
        vc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
        table = torch.randperm(num_pages, device=dev, generator=gen).to(torch.int32).view(batch, pages_per_req)
        slots = i32(list(range(batch)))
        if name in ("attention_decode", "attention_decode_split"):
            q = torch.randn((batch, hq, d), device=dev, generator=gen).bfloat16()
            out = torch.empty_like(q)
            items, tok_req = i32(list(range(batch))), i32(list(range(batch)))
            positions = i32([ctx - 1] * batch)
            if name == "attention_decode":          # the kernel the engine uses: key tiles dealt out evenly
                blocks = ops.decode_balanced_blocks(q.device, batch, hkv, ctx)
                run = lambda: ops.attention_decode_balanced(q, out, kc, vc, items, positions, tok_req, slots, table,
                                                            err, scale=d ** -0.5, window=None, blocks=blocks)
            else:                                   # the same number of splits for every (token, kv head)
                n_splits = ops.decode_splits(batch, hkv, ctx)
                scratch = torch.empty(batch * hq * n_splits * (d + 2), dtype=torch.float32, device=dev)
                run = lambda: ops.attention_decode(q, out, kc, vc, items, positions, tok_req, slots, table, err,
                                                   scale=d ** -0.5, window=None, n_splits=n_splits, scratch=scratch)
            nbytes = 2 * kc.numel() * 2 + 2 * q.numel() * 2
        else:
            qn = min(portion or ctx, ctx)         # query tokens of every request: the end of its context
            q = torch.randn((batch * qn, hq, d), device=dev, generator=gen).bfloat16()
            out = torch.empty_like(q)
            q_start, q_len, kv_len = [r * qn for r in range(batch)], [qn] * batch, [ctx] * batch
            if name == "attention_prefill_mma":
                tiles = [(r, t) for t in reversed(range(-(-qn // 64))) for r in range(batch)]
                tiles_t = i32([x for rt in tiles for x in rt])
                args = (i32(q_start), i32(q_len), i32(kv_len))
                run = lambda: ops.attention_prefill(q, out, kc, vc, tiles_t, *args, slots, table, err,
                                                    scale=d ** -0.5, window=None)
            else:
                records, n_parts, n_split = ops.prefill_tc_records(q_start, q_len, kv_len, list(range(batch)),
                                                                    heads=hq, sms=ops.sm_count(q.device))
                items = ops.PrefillItems(torch.from_numpy(records).to(dev), n_parts, n_split)
                run = lambda: ops.attention_prefill_tc(q, out, kc, vc, items, table, err, scale=d ** -0.5, window=None)
            nbytes = 2 * kc.numel() * 2 + 2 * q.numel() * 2
            flops = batch * 2.0 * 2.0 * (qn * (ctx - qn) + qn * (qn + 1) / 2) * hq * d
    elif name == "rope_kv":
        # q/k norm + rotation + cache write for `batch` tokens of one request (prefill shape)
        n = batch
        pages = -(-n // page)
        kc = torch.zeros((pages, hkv, page, d), dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        qkv = torch.randn((n, (hq + 2 * hkv) * d), device=dev, generator=gen).bfloat16()
        q_out = torch.empty((n, hq, d), dtype=torch.bfloat16, device=dev)
        positions = torch.arange(n, dtype=torch.int32, device=dev)
        tok_req = torch.zeros(n, dtype=torch.int32, device=dev)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        wq, wk = torch.ones(d, device=dev), torch.ones(d, device=dev)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        rot = ops.rope_table(positions, inv_freq)
        slot0, len_n = i32([0]), i32([n])      # made once: a tensor from a host list is a blocking copy
        run = lambda: ops.rope_kv(qkv, q_out, kc, vc, positions, tok_req, slot0, table, wq, wk, rot, err,
                                  n_q_heads=hq, n_kv_heads=hkv, head_dim=d, rotary_dim=d, eps=1e-6,
                                  req_q_len=len_n, req_kv_len=len_n)
        nbytes = qkv.numel() * 2 + q_out.numel() * 2 + 2 * n * hkv * d * 2
    elif name == "sampling":
        # one token per row of float32 logits at the model's vocabulary; --sampling gives temperature,top_k,top_p
        n, vocab = batch, cfg["vocab_size"]
        t_, k_, p_ = sampling if sampling is not None else (0.8, 0, 0.95)
        logits = torch.randn((n, vocab), device=dev, generator=gen) * 3
        out_tok = torch.zeros(n, dtype=torch.int32, device=dev)
        temp = torch.full((n,), float(t_), device=dev)
        top_k = torch.full((n,), int(k_), dtype=torch.int32, device=dev)
        top_p = torch.full((n,), float(p_), device=dev)
        seeds = torch.arange(n, dtype=torch.int64, device=dev)
        counters = torch.zeros(n, dtype=torch.int32, device=dev)
        run = lambda: ops.sample(logits, temp, top_k, top_p, seeds, counters, out_tok)
        nbytes = n * vocab * 4          # one reading of the row; a top-k or top-p threshold reads it four times more each
    elif name == "rmsnorm":
        n, h = batch, cfg["hidden_size"]
        resid = torch.randn((n, h), device=dev, generator=gen)
        delta = torch.randn((n, h), device=dev, generator=gen).bfloat16()
        w = torch.ones(h, device=dev)
        out = torch.empty((n, h), dtype=torch.bfloat16, device=dev)
        run = lambda: ops.add_rmsnorm(resid, delta, w, out, 1e-6)
        nbytes = n * h * (4 + 2 + 4 + 2)
    elif name == "gemm_tc_decode":
        # the engine's own decode product: gate_up of one layer on tcgen05, weight as the row operand
        w = torch.randn((2 * cfg["intermediate_size"], cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        ws = [w.clone() for _ in range(4)]
        x = torch.randn((batch, cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        splits, stages, cluster = ops.swapped_gemm_plan(w.shape[0], w.shape[1], batch)
        out = torch.empty((splits // cluster if cluster > 1 else splits, batch, w.shape[0]),
                          dtype=torch.float32, device=dev)
        turn = [0]
        def run():
            turn[0] = (turn[0] + 1) % len(ws)
            ops.gemm_tc_swapped(ws[turn[0]], x, err, splits, out=out, max_stages=stages, cluster=cluster)
        nbytes = w.numel() * 2
    elif name == "gemm_decode":
        # the library product the decode step uses, for comparison: gate_up of one layer
        w = torch.randn((2 * cfg["intermediate_size"], cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        ws = [w.clone() for _ in range(4)]          # rotate over copies so that L2 holds none of them
        x = torch.randn((batch, cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        turn = [0]
        def run():
            turn[0] = (turn[0] + 1) % len(ws)
            torch.mm(x, ws[turn[0]].t())
        nbytes = w.numel() * 2
    elif name in ("products_chain", "products_separate"):
        # the four products between two attentions of a decode step (output, gate/up, down, the next
        # q|k|v, each with its fused epilogue) for `batch` tokens: as one persistent kernel, or one by one
        h, inter = cfg["hidden_size"], cfg["intermediate_size"]
        mk = lambda *shape, s=1.0: (torch.randn(*shape, device=dev, generator=gen) * s).bfloat16()
        sets = [dict(o=mk(h, hq * d, s=0.02), gu=mk(2 * inter, h, s=0.02), dn=mk(h, inter, s=0.02),
                     qkv=mk((hq + 2 * hkv) * d, h, s=0.02)) for _ in range(3)]      # rotated: none stays in L2
        x0 = mk(batch, hq * d)
        n1, n2 = torch.ones(h, device=dev), torch.ones(h, device=dev)
        qn, kn = torch.ones(d, device=dev), torch.ones(d, device=dev)
        resid = torch.zeros(batch, h, device=dev)
        pages = 4
        kc = torch.zeros((pages, hkv, page, d), dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        q = torch.zeros((batch, hq, d), dtype=torch.bfloat16, device=dev)
        positions = torch.arange(batch, dtype=torch.int32, device=dev) % (pages * page)
        tok_req, slot0 = torch.zeros(batch, dtype=torch.int32, device=dev), i32([0])
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        rot = ops.rope_table(positions, inv_freq)
        plan = lambda w: ops.swapped_gemm_plan(w.shape[0], w.shape[1], batch)
        turn = [0]
        def run():
            turn[0] = (turn[0] + 1) % len(sets)
            w = sets[turn[0]]
            c = ops.ProductChain(batch, err) if name == "products_chain" else None
            resid.zero_()
            s_, st, cl = plan(w["o"])
            xb1, ss1 = ops.gemm_tc_swapped(w["o"], x0, err, s_, max_stages=st, cluster=cl, residual_norm=(resid, n1), chain=c)
            s_, st, cl = plan(w["gu"])
            act = ops.gemm_tc_swapped(w["gu"], xb1, err, s_, max_stages=st, cluster=cl, swiglu=True,
                                      colscale=(ss1, h, 1e-6), chain=c)
            s_, st, cl = plan(w["dn"])
            xb2, ss2 = ops.gemm_tc_swapped(w["dn"], act, err, s_, max_stages=st, cluster=cl, residual_norm=(resid, n2), chain=c)
            s_, st, cl = plan(w["qkv"])
            ops.gemm_qkv_rope(w["qkv"], xb2, err, s_, q, kc, vc, positions, tok_req, slot0, table, qn, kn, rot,
                              n_q_heads=hq, n_kv_heads=hkv, eps=1e-6, max_stages=st, colscale=(ss2, h, 1e-6), chain=c)
            ops.flush_chains()
        nbytes = sum(t.numel() * 2 for t in sets[0].values())
    elif name in ("gemm_pair_swiglu", "gemm_prefill_library"):
        # the prefill gate/up product of one layer over ctx tokens with the activation: the engine's
        # kernel on pairs of SMs with the activation in its epilogue, or the library product followed
        # by the activation kernel
        inter, hidden = cfg["intermediate_size"], cfg["hidden_size"]
        w = (torch.randn((2 * inter, hidden), device=dev, generator=gen) * 0.02).bfloat16()
        x = torch.randn((ctx, hidden), device=dev, generator=gen).bfloat16()
        act = torch.empty((ctx, inter), device=dev, dtype=torch.bfloat16)
        if name == "gemm_pair_swiglu":
            run = lambda: ops.gemm_pair(x, w, err, swiglu=True)
        else:
            def run():
                ops.swiglu(torch.mm(x, w.t()), act, block=ops.SWIGLU_TILE_BLOCK)
        nbytes = (w.numel() + x.numel() + act.numel()) * 2
        flops = 2.0 * ctx * 2 * inter * hidden
    else:
        raise SystemExit(f"unknown kernel case {name!r}")
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        run()
    end.record()
    torch.cuda.synchronize()
    us = begin.elapsed_time(end) * 1e3 / iters
    gbs = nbytes / (us * 1e-6) / 1e9
    res = {"kernel": name, "batch": batch, "ctx": ctx, "us": round(us, 2), "bytes": nbytes,
           "GB/s": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4), "peaks": peaks["source"]}
    if flops:
        tf = flops / (us * 1e-6) / 1e12
        res.update({"TFLOP/s": round(tf, 1), "bf16_frac": round(tf / peaks["bf16_tflops"], 4)})
    assert err.tolist()[0] == 0
    return res


def prefill_attention_timeline(batch: int, ctx: int, portion: int, sizes: str) -> int:
    """Time stamps of the roles of the persistent prefill attention kernel on a few SMs (the library must
    have been built with TOKAMAK_B200_NVCC_FLAGS=-DTK_TIMELINE): when the producer published an item, when
    the softmax warps of query tile 0 / 1 started it, ended its key tiles, saw the last product and had
    written their rows, and the stamps of one block's thread per role within the key tiles."""
    import torch
    from tokamak_b200.csrc import ops
    cfg = SIZES[sizes][1] if sizes in SIZES else QWEN3_8B
    hq, hkv, d, page = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], 16
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(0)
    pages_per_req = -(-ctx // page)
    num_pages = batch * pages_per_req
    kc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
    vc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
    table = torch.randperm(num_pages, device=dev, generator=gen).to(torch.int32).view(batch, pages_per_req)
    qn = min(portion or ctx, ctx)
    q = torch.randn((batch * qn, hq, d), device=dev, generator=gen).bfloat16()
    out = torch.empty_like(q)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    records, n_parts, n_split = ops.prefill_tc_records([r * qn for r in range(batch)], [qn] * batch, [ctx] * batch,
                                                        list(range(batch)), heads=hq, sms=ops.sm_count(q.device))
    items = ops.PrefillItems(torch.from_numpy(records).to(dev), n_parts, n_split)
    run = lambda: ops.attention_prefill_tc(q, out, kc, vc, items, table, err, scale=d ** -0.5, window=None)
    for _ in range(3):
        run()
    buf = ops.timeline_start(1 << 16)
    torch.cuda.synchronize()
    run()
    torch.cuda.synchronize()
    buf[0] = (buf.numel() - 1) // 2          # the roles' own ranges lie at the buffer's end
    every = [r for r in ops.timeline_read(buf) if r[0] > 0]
    recs = [r for r in every if r[1] == 30]
    clocks = [0] * 9
    for _, kernel, phase, _, value in every:
        if kernel == 32 and phase < 9:
            clocks[phase] += value
    if err.tolist()[0] != 0 or not recs:
        print("error word", err.tolist(), "records", len(recs))
        return 1
    t0 = recs[0][0]
    lengths = [int(r[5] - r[4]) for r in records]
    what = {1: "published", 10: "tile 0 starts", 11: "tile 1 starts", 20: "tile 0 keys done", 21: "tile 1 keys done",
            30: "tile 0 last product", 31: "tile 1 last product", 40: "tile 0 written", 41: "tile 1 written",
            50: "tile 0 parts added up", 51: "tile 1 parts added up", 60: "issuer 0 has item", 61: "issuer 1 has item"}
    coarse = [r for r in recs if r[2] < 70]
    by_sm: dict = {}
    for t, _, ph, sm, val in coarse:
        by_sm.setdefault(sm, []).append(((t - t0) / 1e3, ph, val))
    ends = sorted(max(x[0] for x in v) for v in by_sm.values())
    print(f"{batch} x {qn} tokens at the end of {ctx}, {hq} heads: {len(records)} records, {n_split} blocks of tokens cut; "
          f"blocks end after {ends[0]:.1f} / {ends[len(ends) // 2]:.1f} / {ends[-1]:.1f} us (first / median / last)")
    for sm in sorted(by_sm)[1:3]:
        print(f"SM {sm}")
        for t, ph, val in by_sm[sm]:
            n_rec = val // hq
            tiles = lengths[n_rec] if n_rec < len(lengths) else 0
            print(f"  {t:8.2f} us  item {val:5d} ({tiles:3d} key tiles)  {what.get(ph, ph)}")
    if clocks[8]:
        parts = ["waiting for S", "S loaded", "maximum", "exponentials, sum, conversion, store issued", "store arrived",
                 "fence and arrival", "loop", "between items"]
        print(f"one softmax thread of each query tile of block 0, clocks per key tile ({clocks[8]} key tiles):")
        for name, c in zip(parts, clocks):
            print(f"  {c / clocks[8]:7.1f}  {name}")
    fine = {70: "scores seen", 74: "probabilities given", 82: "S issued", 84: "probabilities seen", 86: "O += P V issued"}
    print("one block, within its key tiles (the stamps of this block cost it a few percent)")
    for t, _, ph, sm, val in [r for r in recs if r[2] >= 70][:64]:
        print(f"  {(t - t0) / 1e3:8.2f} us  tile {ph & 1}  {fine.get(ph - (ph & 1), ph):20s} key tile {val}")
    return 0


def tcgen05_probe() -> int:
    """Two tables of what the hardware gives the tcgen05 kernels (csrc/tcgen05_probe.cu): the cost of
    issuing a tcgen05.mma by shape, operand source and number of issuing threads, and the clocks one
    softmax warp of the prefill attention kernel needs for a 64-key tile in several forms of its loop."""
    from tokamak_b200.csrc import ops
    print("tcgen05.mma M 128 x N x K 16, bfloat16, 96 in a row: clocks per product until issued / until done")
    modes = {0: "one thread, A and B in shared memory", 1: "one thread, A in tensor memory",
             2: "two threads, A and B in shared memory", 3: "two threads, A in tensor memory",
             4: "one thread, 8 x (N, shared) then 4 x (N 128, A in tensor memory)"}
    for mode, name in modes.items():
        for n in (16, 64, 128, 256):
            if n > 128 and mode in (2, 3, 4) or mode == 4 and n == 16:
                continue
            for _ in range(2):
                rows = ops.probe_mma_issue(mode, n)
            cells = " | ".join(f"{r['issue_clk']:6.1f} / {r['done_clk']:6.1f} clk ({r['done_ns']:5.1f} ns)" for r in rows)
            print(f"  {name:66s} N {n:3d}: {cells}")
    print("one softmax warp, 64 keys: clocks per tile (load, maximum, exponentials + conversion + store, store arrived, fence)")
    forms = {0: "as the kernel has it", 1: "four chains for the maximum", 2: "second half loaded under the first maximum",
             3: "four chains and the split load", 4: "1 exponential in 4 by polynomial", 5: "2 in 4 by polynomial",
             6: "all by polynomial"}
    for variant, name in forms.items():
        for wg in (1, 2):
            for _ in range(2):
                r = ops.probe_softmax_tile(variant, wg)
            print(f"  {name:44s} {wg} warp(s) per scheduler: {r['tile']:7.1f}  ({r['load']:.0f}, {r['maximum']:.0f}, "
                  f"{r['exponentials_store']:.0f}, {r['store_arrived']:.0f}, {r['fence']:.0f})")
    return 0


def decode_timeline(batch: int, layers: int, ctx: int) -> int:
    """Lay the blocks of every kernel of two decode steps out on one time axis (the library must have
    been built with time stamps: TOKAMAK_B200_NVCC_FLAGS=-DTK_TIMELINE, see csrc/timeline.cuh).
    Prints, per kernel instance, when its blocks started, were released by the kernel before, finished
    their products and ended, in microseconds from the first stamp."""
    import torch
    from tokamak_b200.csrc import ops
    from tokamak_b200.engine.core import random_core
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    raw = dict(QWEN3_8B, num_hidden_layers=layers)
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=ctx, page_size=16,
                       pool_tokens=batch * ctx, max_slots=batch, max_step_tokens=2048)
    step = core.step
    ids = [f"r{i}" for i in range(batch)]
    for r in ids:
        step.admit(r, SamplingRow())
    fill_context(core, ids, ctx - 40, raw["vocab_size"], seed=1)
    step.run_and_sample([StepEntry(r, [1 + i], [0]) for i, r in enumerate(ids)])
    entries = [StepEntry(r, None, [0]) for r in ids]
    for _ in range(6):
        step.run_and_sample(entries)
    buf = ops.timeline_start(1 << 18)
    first, second = step.launch_and_sample(entries), step.launch_and_sample(entries)
    step.collect(first); step.collect(second)
    recs = ops.timeline_read(buf)
    names = {1: "begin", 2: "attention", 3: "sample", 4: "embed", 10: "product", 11: "product+swiglu",
             12: "product+residual", 13: "q|k|v+rope", 20: "chain"}
    t0 = recs[0][0]
    by_kernel: dict = {}
    for t, k, ph, sm, blk in recs:
        by_kernel.setdefault(k, []).append((t - t0, ph))
    instances = []
    for k, rows in by_kernel.items():
        if k not in names:
            continue
        cur, last_start = None, None
        for t, ph in sorted(rows):
            if ph == 0 and (last_start is None or t - last_start > 4000):     # a gap of 4 us: another launch
                cur = {"k": k, "ph": {}}
                instances.append(cur)
            if ph == 0:
                last_start = t
            if cur is not None:
                cur["ph"].setdefault(ph, []).append(t)
    instances.sort(key=lambda i: min(i["ph"][0]))
    rng = lambda v: f"{min(v) / 1e3:7.1f}-{max(v) / 1e3:7.1f}" if v else " " * 15
    print(f"batch {batch}, {layers} layers of Qwen3-8B sizes, context {ctx}: two decode steps, us from the first stamp")
    print(f"{'kernel':17s} {'blocks':>6s} {'started':>15s} {'released':>15s} {'products done':>15s} {'ended':>15s}")
    for i in instances:
        ph = i["ph"]
        done = ph.get(2, []) if i["k"] != 20 else [t for q in ph if 31 <= q < 40 for t in ph[q]]
        print(f"{names[i['k']]:17s} {len(ph[0]):6d} {rng(ph.get(0))} {rng(ph.get(1))} {rng(done)} {rng(ph.get(4))}")
    return 0


def reference_main(args) -> int:
    """``--impl reference``: the unmodified reference from ``baseline/_ref`` on the same metric, or
    one line that says why it cannot run.  Everything it does is in ``baseline/reference_arm.py``."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm
    why = reference_arm.available()
    if why is None and args.gpus != 1:
        why = "the reference runs on one GPU only"
    if why is None and args.sizes not in SIZES:
        why = "--sizes 0.6b is for --workload throughput only"
    if why is not None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    model_name, sizes = SIZES[args.sizes]
    raw = dict(sizes)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    try:
        config = bench_config(model_name, raw, sizes["num_hidden_layers"], args.batch, args.seq_len,
                              args.prefill_tokens, load_peaks()["source"])
        line = reference_arm.run(raw, model_name, args.batch, args.seq_len, args.prefill_tokens, max(1, args.steps),
                                 max(3, args.warmup), points=() if args.skip_points else tuple(args.points),
                                 clock_sampler=ClockSampler(0), config=config)
    except Exception as err:    # the reference's failure is reported, never hidden behind our numbers
        print(json.dumps({"impl": "reference", "unavailable": f"{type(err).__name__}: {str(err)[:300]}"}))
        return 0
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the 36 of Qwen3-8B")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out the further batch sizes")
    ap.add_argument("--points", type=lambda v: [int(x) for x in v.split(",") if x], default=[1, 64],
                    help="further decode batch sizes to time, comma-separated (default 1,64)")
    ap.add_argument("--sampling", default=None,
                    type=lambda v: tuple(float(x) for x in v.split(",")) if v else None,
                    help="temperature,top_k,top_p of the timed decode steps of the main batch (default: greedy), "
                         "e.g. 0.8,0,0.95; the points and the end-to-end run stay greedy")
    ap.add_argument("--kernel", default=None, help="time one kernel alone instead: attention_decode, attention_decode_split, "
                    "attention_prefill (tcgen05), attention_prefill_mma, rope_kv, rmsnorm, sampling (--batch rows, --sampling T,K,P), gemm_tc_decode, gemm_decode (library), "
                    "gemm_pair_swiglu, gemm_prefill_library (--ctx tokens), products_chain / products_separate (the four products "
                    "between two attentions of a decode step, as one kernel or one by one); attention_prefill_timeline prints the time stamps of the persistent prefill attention kernel's roles; tcgen05_probe prints what issuing a tcgen05.mma costs by shape and what a softmax warp needs for a key tile; decode_timeline prints when the blocks of every "
                    "kernel of a decode step run (needs a library built with TOKAMAK_B200_NVCC_FLAGS=-DTK_TIMELINE)")
    ap.add_argument("--ctx", type=int, default=CONTEXT, help="context length of a --kernel case")
    ap.add_argument("--workload", default=None, choices=["throughput", "latency", "mixed"],
                    help="run the reference's throughput workload through LLM.generate, or its single-sequence "
                         "latency measurement (512 prompt tokens, 128 greedy steps), or a mixed batch of 32 "
                         "requests (prompts of 128 to 4,096 tokens in portions of 512 beside decode tokens, 256 "
                         "new tokens each; --sizes 14b is the configuration it is named for), instead")
    ap.add_argument("--prefill-chunk", type=int, default=512, help="portion size of --workload mixed")
    ap.add_argument("--portion", type=int, default=0,
                    help="query tokens per request of the attention_prefill kernel cases (the end of a context "
                         "of --ctx tokens; default: the whole context)")
    ap.add_argument("--sizes", default="8b", choices=["0.6b", "8b", "14b", "32b"],
                    help="layer sizes: of --workload (0.6b, 8b), or of the decode/prefill run (8b, the metric's "
                         "own, 14b, 32b)")
    ap.add_argument("--num-requests", type=int, default=32)
    ap.add_argument("--max-new-cap", type=int, default=256)
    ap.add_argument("--kv-pool-tokens", type=int, default=16384)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--seq-len", type=int, default=CONTEXT, help="context length at which the decode steps run")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="length of the timed prompt")
    ap.add_argument("--prompt-tokens", type=int, default=None,
                    help="length of the random prompts (and prompt portions) that fill the contexts before the "
                         "decode steps are timed (default: --prefill-tokens)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_main(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if args.kernel == "decode_timeline":
        return decode_timeline(args.batch, args.layers or 3, args.ctx)
    if args.kernel == "tcgen05_probe":
        return tcgen05_probe()
    if args.kernel == "attention_prefill_timeline":
        return prefill_attention_timeline(args.batch, args.ctx, args.portion, args.sizes)
    if args.kernel:
        print(json.dumps(kernel_case(args.kernel, args.batch, args.ctx, steps, load_peaks(), args.portion, args.sizes,
                                     args.sampling)))
        return 0
    if args.workload == "latency":
        print(json.dumps(latency_workload(args.sizes, 512, 128, 3, args.seed)))
        return 0
    if args.workload == "mixed":
        print(json.dumps(mixed_workload(args.sizes, args.num_requests, args.max_new_cap, args.prefill_chunk,
                                        args.seed)))
        return 0
    if args.workload == "throughput":
        print(json.dumps(throughput_workload(args.sizes, args.num_requests, args.max_new_cap, args.batch,
                                             args.kv_pool_tokens, args.seed)))
        return 0

    import torch
    from tokamak_b200.engine.core import random_core

    if args.sizes not in SIZES:
        raise SystemExit("--sizes 0.6b is for --workload throughput only")
    model_name, sizes = SIZES[args.sizes]
    raw = dict(sizes)
    n_layers = args.layers or raw["num_hidden_layers"]
    raw["num_hidden_layers"] = n_layers
    vocab = raw["vocab_size"]
    peaks = load_peaks()
    ctx, pf_tokens = args.seq_len, args.prefill_tokens      # the defaults unless asked otherwise
    global PROMPT_PORTION
    PROMPT_PORTION = args.prompt_tokens or pf_tokens
    max_batch = max([args.batch, 1] + ([] if args.skip_points else list(args.points)))
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=max(ctx, pf_tokens), page_size=16,
                       pool_tokens=max(max_batch * ctx, pf_tokens + 64), max_slots=max_batch,
                       max_step_tokens=max(pf_tokens, args.batch * ctx))
    wbytes = weight_bytes(core)

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    main_run = time_decode(core, args.batch, steps, warmup, ctx, vocab, args.sampling)
    prefill_ms = time_prefill(core, vocab, pf_tokens)
    points = {}
    checked = main_run["checked"]
    if not args.skip_points:
        for b in args.points:
            run = time_decode(core, b, steps, warmup, ctx, vocab)
            points[f"decode_b{b}"] = round(run["tok_s"], 1)
            checked = checked and run["checked"]
    e2e = time_e2e(core, args.batch, steps, warmup, ctx, vocab)
    clocks = sampler.stop()

    step_bytes = wbytes + main_run["kv_bytes"]
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    pf_flops = step_flops(raw, n_layers, pf_tokens)
    pf_frac = pf_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name} layer sizes, context {ctx})",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), uniform random token ids",
        "config": bench_config(model_name, raw, sizes["num_hidden_layers"], args.batch, ctx, pf_tokens,
                               peaks["source"]),
        "prompt_tokens": PROMPT_PORTION,
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(pf_tokens / (prefill_ms / 1e3), 1), "tokens": pf_tokens,
                    "ms": round(prefill_ms, 3), "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
        "host_ms_per_step": round(main_run["wall_ms_per_step"], 4),
        # every timed decode step's tokens equal those of the same steps run again kernel by kernel
        # (no CUDA graph, no step launched ahead, tokens fed by the host)
        "checked": checked,
        "device_step_h2d_bytes": round(main_run["h2d_bytes_per_step"], 1),
    }
    print(json.dumps(line))
    if not checked:
        print("bench.py: the timed decode steps produced other tokens than the same steps run "
              "kernel by kernel", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
