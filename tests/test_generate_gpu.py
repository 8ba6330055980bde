"""Generation through the Python entry point against the plain implementation."""

from __future__ import annotations

import dataclasses

import pytest
import torch

import tiny_configs
from helpers import model_folder, plain_logits, random_tokens
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def llm_for(tag, dtype, **kw):
    from tokamak_b200 import LLM
    kw.setdefault("block_size", tiny_configs.ALL[tag][2])
    return LLM(model_folder(tag, dtype), dtype=dtype, **kw)


def prompts_for(tag, lengths):
    vocab = tiny_configs.ALL[tag][0]["vocab_size"]
    return [random_tokens(vocab, n, seed=7 * n + 1) for n in lengths]


def test_greedy_matches_plain_float32():
    """Configuration A's workload: prompts of 5, 17 and 33 tokens, 8 greedy tokens each."""
    from tokamak_b200 import SamplingParams
    llm = llm_for("A", "float32")
    prompts = prompts_for("A", [5, 17, 33])
    outs = llm.generate(prompt_token_ids=prompts,
                        sampling_params=SamplingParams(temperature=0.0, max_new_tokens=8))
    cfg, w = plain.load_folder(model_folder("A", "float32"))
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 8)
        assert o.finish_reason.value == "length" and o.prompt_token_ids == p
    assert [o.request_id for o in outs] == [0, 1, 2]
    assert all(0 < o.ttft_s <= o.latency_s for o in outs)


def test_chunked_prefill_with_temperature_matches_plain_float32():
    """Configuration B's workload: prompts of 1/7/31/64/100, portions of 24 beside decodes,
    temperature 0.8, seed 1, 12 new tokens.  Every token must be the plain sampler's draw
    from the plain logits of the same prefix."""
    from tokamak_b200 import SamplingParams
    llm = llm_for("B", "float32", prefill_chunk=24, max_num_batched_tokens=48, max_batch_size=4)
    prompts = prompts_for("B", [1, 7, 31, 64, 100])
    params = SamplingParams(temperature=0.8, seed=1, max_new_tokens=12)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert llm.last_stats["mixed_steps"] > 0
    folder = model_folder("B", "float32")
    for p, o in zip(prompts, outs):
        assert len(o.output_token_ids) == 12
        seq = list(p)
        for i, tok in enumerate(o.output_token_ids):
            logits = plain_logits(folder, seq)[-1]
            assert tok == plain.sample_token(logits.float(), 0.8, seed=1, token_index=i), (len(p), i)
            seq.append(tok)


def test_preemption_is_invisible_in_greedy_tokens():
    """A pool so small that sequences are evicted and recomputed gives the same tokens as a
    large pool (after the reference's tests/integration/test_generate_e2e.py:180-213)."""
    from tokamak_b200 import SamplingParams
    prompts = prompts_for("A", [20, 28, 24, 30])
    params = SamplingParams(temperature=0.0, max_new_tokens=24)
    big = llm_for("A", "float32", max_seq_len=64, kv_pool_tokens=1024)
    want = [o.output_token_ids for o in big.generate(prompt_token_ids=prompts, sampling_params=params)]
    assert big.last_stats["preemptions"] == 0
    small = llm_for("A", "float32", max_seq_len=64, kv_pool_tokens=128)
    outs = small.generate(prompt_token_ids=prompts, sampling_params=params)
    assert small.last_stats["preemptions"] > 0
    assert [o.output_token_ids for o in outs] == want
    assert sum(o.num_preemptions for o in outs) == small.last_stats["preemptions"]
    # four requests in four slots: every record holds, after all the evictions, as many draws as
    # its request sampled tokens, and the position its request reached
    records = small.core.cache.slot_records[:4].cpu()         # the first four slots are handed out first
    assert records[:, 1].tolist() == [24] * 4
    assert sorted(records[:, 0].tolist()) == sorted(len(p) + 23 for p in prompts)
    small.cache_manager.check_invariants()
    assert all(g.num_free == g.num_pages for g in small.cache_manager.kv_groups)


def test_seeded_sampling_is_reproducible_and_independent_of_batching():
    from tokamak_b200 import SamplingParams
    prompts = prompts_for("B", [9, 30, 12, 21])
    params = [SamplingParams(temperature=1.0, top_k=20, top_p=0.9, seed=40 + i, max_new_tokens=10)
              for i in range(4)]
    a = llm_for("B", "float32", max_batch_size=4).generate(prompt_token_ids=prompts, sampling_params=params)
    b = llm_for("B", "float32", max_batch_size=1).generate(prompt_token_ids=prompts, sampling_params=params)
    c = llm_for("B", "float32", max_batch_size=4, prefill_chunk=5, max_num_batched_tokens=11).generate(
        prompt_token_ids=prompts, sampling_params=params)
    toks = lambda outs: [o.output_token_ids for o in outs]
    assert toks(a) == toks(b) == toks(c)
    assert len({tuple(t) for t in toks(a)}) == 4


def test_finishing_rules_and_errors():
    from tokamak_b200 import LLM, SamplingParams
    llm = llm_for("A", "float32", max_seq_len=40)
    p = prompts_for("A", [10])[0]
    first = llm.generate(prompt_token_ids=[p], sampling_params=SamplingParams(temperature=0.0, max_new_tokens=3))
    assert len(first[0].output_token_ids) == 3 and first[0].finish_reason.value == "length"
    # treat the second generated token as EOS
    eos = first[0].output_token_ids[1]
    llm.model_config = dataclasses.replace(llm.model_config, eos_token_ids=(eos,))
    stop = llm.generate(prompt_token_ids=[p], sampling_params=SamplingParams(temperature=0.0, max_new_tokens=9))
    assert stop[0].finish_reason.value == "stop" and stop[0].output_token_ids[-1] == eos
    assert len(stop[0].output_token_ids) <= 2
    on = llm.generate(prompt_token_ids=[p], sampling_params=SamplingParams(temperature=0.0, max_new_tokens=9,
                                                                          ignore_eos=True))
    assert len(on[0].output_token_ids) == 9
    llm.model_config = dataclasses.replace(llm.model_config, eos_token_ids=())
    ctx = llm.generate(prompt_token_ids=[p], sampling_params=SamplingParams(temperature=0.0, max_new_tokens=500))
    assert len(ctx[0].output_token_ids) == 30 and ctx[0].finish_reason.value == "length"   # max_seq_len 40
    with pytest.raises(ValueError, match="does not fit"):
        llm.generate(prompt_token_ids=[list(range(40))])
    with pytest.raises(ValueError, match="exactly one"):
        llm.generate()
    with pytest.raises(ValueError, match="SamplingParams for"):
        llm.generate(prompt_token_ids=[p, p], sampling_params=[SamplingParams()])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        llm.generate(prompt_token_ids=[[1, 999999]])
    with pytest.raises(ValueError, match="kv_pool_tokens"):
        LLM(model_folder("A", "float32"), dtype="float32", max_seq_len=64, kv_pool_tokens=32)
    with pytest.raises(ValueError, match="Unknown dtype"):
        LLM(model_folder("A", "float32"), dtype="float16")


@pytest.mark.parametrize("tag", ["A", "B"])
def test_greedy_bfloat16_picks_a_top_token(tag):
    """In bfloat16 near-ties may flip, so tokens are judged against the plain logits: each
    generated token must be within a small margin of the plain maximum for its prefix."""
    from tokamak_b200 import SamplingParams
    llm = llm_for(tag, "bfloat16", prefill_chunk=16, max_num_batched_tokens=40)
    prompts = prompts_for(tag, [6, 19, 45])
    outs = llm.generate(prompt_token_ids=prompts,
                        sampling_params=SamplingParams(temperature=0.0, max_new_tokens=8))
    folder = model_folder(tag, "bfloat16")
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.output_token_ids:
            logits = plain_logits(folder, seq)[-1]
            assert logits[tok] >= logits.max() - 0.04 * logits.std()
            seq.append(tok)


def test_window_policy_matches_a_windowed_config():
    """attention_policy='window:W' equals a config.json that windows every layer."""
    from tokamak_b200 import SamplingParams
    llm = llm_for("A", "float32", attention_policy="window:12")
    prompts = prompts_for("A", [40])
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=6))
    cfg, w = plain.load_folder(model_folder("A", "float32"))
    cfg = dict(cfg, use_sliding_window=True, sliding_window=12, max_window_layers=0)
    assert outs[0].output_token_ids == plain.greedy_generate(cfg, w, prompts[0], 6)
    with pytest.raises(ValueError, match="attention_policy"):
        llm_for("A", "float32", attention_policy="streaming:8+2")


def test_many_requests_small_pool_equal_single_request_runs():
    """Forty requests of mixed lengths and sampling settings through a pool that forces waiting
    and preemption: every request's tokens equal those of the same request run alone."""
    from tokamak_b200 import SamplingParams
    lengths = [3 + (i * 37) % 90 for i in range(40)]
    prompts = prompts_for("C", lengths)
    params = [SamplingParams(temperature=0.0 if i % 3 else 0.9, top_k=0 if i % 2 else 12, seed=100 + i,
                             max_new_tokens=4 + i % 9) for i in range(40)]
    shared = llm_for("C", "float32", max_seq_len=128, kv_pool_tokens=512, max_batch_size=6,
                     max_num_batched_tokens=96, prefill_chunk=40)
    outs = shared.generate(prompt_token_ids=prompts, sampling_params=params)
    stats = shared.last_stats
    assert stats["mixed_steps"] > 0 and stats["decode_tokens"] > 0
    shared.cache_manager.check_invariants()
    assert all(g.num_free == g.num_pages for g in shared.cache_manager.kv_groups)
    alone = llm_for("C", "float32", max_seq_len=128, kv_pool_tokens=128, max_batch_size=1)
    for i in range(0, 40, 3):
        want = alone.generate(prompt_token_ids=[prompts[i]], sampling_params=params[i])[0]
        assert outs[i].output_token_ids == want.output_token_ids, i
        assert len(outs[i].output_token_ids) == params[i].max_new_tokens


def test_steps_launched_ahead_end_where_the_requests_end_alone():
    """Decode steps are launched before the step before them has been read.  Requests that stop
    on an end-of-sequence token, or at different lengths, while such a step is already running
    end exactly where they end alone, and every page and slot comes back."""
    from tokamak_b200 import SamplingParams
    llm = llm_for("A", "float32", max_batch_size=4)
    prompts = prompts_for("A", [6, 11, 19, 8])
    free_run = SamplingParams(temperature=0.0, max_new_tokens=20)
    alone = [llm.generate(prompt_token_ids=[p], sampling_params=free_run)[0].output_token_ids for p in prompts]
    eos = alone[1][7]
    limits = [20, 20, 13, 5]
    want = []
    for toks, limit in zip(alone, limits):
        toks = toks[:limit]
        want.append(toks[:toks.index(eos) + 1] if eos in toks else toks)
    llm.model_config = dataclasses.replace(llm.model_config, eos_token_ids=(eos,))
    params = [SamplingParams(temperature=0.0, max_new_tokens=n) for n in limits]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert [o.output_token_ids for o in outs] == want
    assert outs[1].finish_reason.value == "stop" and len(outs[1].output_token_ids) <= 8
    assert outs[3].finish_reason.value in ("length", "stop")
    assert llm.last_stats["decode_steps"] >= 10
    llm.cache_manager.check_invariants()
    assert all(g.num_free == g.num_pages for g in llm.cache_manager.kv_groups)
    assert llm.cache_manager.num_free_slots == llm.cache_manager.max_slots


def test_portions_and_admissions_launched_ahead_end_where_the_requests_end_alone():
    """Every kind of step is launched before the step before it has been read: prompt portions
    go on, requests are admitted, and the tokens that the step in flight samples are fed on the
    device.  Six requests through two slots, prompts cut into portions of five, one request
    stopping on an end-of-sequence token while the step after is already running: all end
    exactly where they end alone, step by step with nothing launched ahead, and every page and
    slot comes back."""
    from tokamak_b200 import SamplingParams
    llm = llm_for("A", "float32", max_batch_size=2, prefill_chunk=5, max_num_batched_tokens=9, max_seq_len=64, kv_pool_tokens=64)
    prompts = prompts_for("A", [6, 11, 19, 8, 3, 14])
    free_run = SamplingParams(temperature=0.0, max_new_tokens=16)
    llm.plain_steps = True
    alone = [llm.generate(prompt_token_ids=[p], sampling_params=free_run)[0].output_token_ids for p in prompts]
    assert llm.last_stats["steps_launched_ahead"] == 0
    eos = alone[2][5]
    limits = [16, 9, 16, 4, 12, 16]
    want = []
    for toks, limit in zip(alone, limits):
        toks = toks[:limit]
        want.append(toks[:toks.index(eos) + 1] if eos in toks else toks)
    llm.model_config = dataclasses.replace(llm.model_config, eos_token_ids=(eos,))
    params = [SamplingParams(temperature=0.0, max_new_tokens=n) for n in limits]
    llm.plain_steps = False
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    stats = llm.last_stats
    assert [o.output_token_ids for o in outs] == want
    assert outs[2].finish_reason.value == "stop"
    assert stats["portions_launched_ahead"] >= 6 and stats["steps_launched_ahead"] >= stats["steps"] // 2
    llm.cache_manager.check_invariants()
    assert all(g.num_free == g.num_pages for g in llm.cache_manager.kv_groups)
    assert llm.cache_manager.num_free_slots == llm.cache_manager.max_slots


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_launched_ahead_equal_the_same_workloads_step_by_step(seed):
    """Random requests (lengths, limits, greedy or seeded sampling, an end-of-sequence token that some
    of them meet) through random engine settings (slots, token budget, portion size, a pool that makes
    requests wait or be preempted): with every step launched ahead of the read of the step before it
    the requests end token for token as with plain steps, and nothing is left held."""
    import random
    from tokamak_b200 import SamplingParams
    rng = random.Random(1000 + seed)
    tag = "BC"[seed % 2]
    vocab = tiny_configs.ALL[tag][0]["vocab_size"]
    n_req = rng.randint(5, 12)
    lengths = [rng.randint(2, 70) for _ in range(n_req)]
    prompts = [random_tokens(vocab, n, seed=seed * 100 + i) for i, n in enumerate(lengths)]
    params = [SamplingParams(temperature=rng.choice([0.0, 0.0, 0.8]), top_k=rng.choice([0, 8]), top_p=rng.choice([1.0, 0.9]),
                             seed=seed * 1000 + i, max_new_tokens=rng.randint(1, 24)) for i in range(n_req)]
    chunk = rng.choice([3, 8, 33])
    settings = dict(max_seq_len=96, kv_pool_tokens=rng.choice([96, 160, 384]), max_batch_size=rng.randint(1, 5),
                    max_num_batched_tokens=chunk + rng.randint(2, 12), prefill_chunk=chunk,
                    step_token_multiple=rng.choice([1, 4, 128]))
    llm = llm_for(tag, "float32", **settings)
    llm.plain_steps = True
    free = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    # an end-of-sequence token that at least one request produces in the middle of its run
    long_runs = [o.output_token_ids for o in free if len(o.output_token_ids) >= 4]
    if long_runs:
        eos = rng.choice(long_runs)[2]
        llm.model_config = dataclasses.replace(llm.model_config, eos_token_ids=(eos,))
    want = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert llm.last_stats["steps_launched_ahead"] == 0
    llm.plain_steps = False
    got = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert [o.output_token_ids for o in got] == [o.output_token_ids for o in want], settings
    assert [o.finish_reason for o in got] == [o.finish_reason for o in want]
    assert llm.last_stats["steps_launched_ahead"] > 0
    llm.cache_manager.check_invariants()
    assert all(g.num_free == g.num_pages for g in llm.cache_manager.kv_groups)
    assert llm.cache_manager.num_free_slots == llm.cache_manager.max_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_driven_by_the_slot_records_equal_steps_laid_out_by_the_host(dtype):
    """Steps of single next tokens whose tokens, positions, sampling parameters and generator
    counters come from the slot records on the device (two steps in flight, requests in a
    changing order, with and without CUDA graphs, also mixed with a request that brings its
    tokens itself) against steps in which the host brings every token and every counter:
    the same tokens, and records that hold what happened."""
    from tokamak_b200.engine.replay import build_core
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    tag = "C" if dtype == "bfloat16" else "B"
    cfg, _, page = tiny_configs.ALL[tag][:3]
    core = build_core(model_folder(tag, dtype), dtype, max_tokens=512, page_size=page)
    step = core.step
    prompts = [random_tokens(cfg["vocab_size"], n, seed=n) for n in (9, 4, 17)]
    rows = lambda k: [SamplingRow(0.7, 0, 1.0, seed=100 + i, counter=k) for i in range(3)]
    steps = 12

    def by_host(ids):
        toks = step.run_and_sample([StepEntry(r, p, [len(p) - 1]) for r, p in zip(ids, prompts)], rows(0))
        out = [toks]
        for k in range(1, steps):
            toks = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)], rows(k))
            out.append(toks)
        for r in ids:
            step.free(r)
        return out

    def by_device(ids, extra=None):
        for r, row in zip(ids, rows(0)):
            step.admit(r, row)                         # the records are written once, here
        flight = step.launch_and_sample([StepEntry(r, p, [len(p) - 1]) for r, p in zip(ids, prompts)])
        out, order_before = [], [0, 1, 2]
        for k in range(1, steps):
            order = [2, 0, 1] if k % 2 else [0, 1, 2]  # the list of slots changes from step to step
            entries = [StepEntry(ids[i], None, [0]) for i in order]
            if extra is not None and k == 5:           # a prompt portion rides along: a laid-out step
                entries.append(StepEntry(extra, prompts[1], []))
            ahead = step.launch_and_sample(entries)
            toks = step.collect(flight)
            out.append([toks[order_before.index(i)] for i in range(3)])
            flight, order_before = ahead, order
        toks = step.collect(flight)
        out.append([toks[order_before.index(i)] for i in range(3)])
        for i, r in enumerate(ids):
            rec = step.record(r)
            assert rec["counter"] == steps and rec["last_token"] == out[-1][i]
            assert rec["num_computed"] == len(prompts[i]) + steps - 1 == step.length(r)
            assert rec["seed"] == 100 + i and abs(rec["temperature"] - 0.7) < 1e-6
        for r in ids + ([extra] if extra else []):
            step.free(r)
        return out

    want = by_host(["h0", "h1", "h2"])
    replays = step.graph_replays
    assert by_device(["d0", "d1", "d2"]) == want          # shapes seen once or twice: mostly kernel by kernel
    assert by_device(["e0", "e1", "e2"]) == want          # replayed from the captured graph
    assert step.graph_replays > replays
    assert by_device(["f0", "f1", "f2"], extra="x") == want
    # a steady step copies nothing to the device but new pages: far less than a laid-out step would
    step.admit("s", SamplingRow())
    step.run_and_sample([StepEntry("s", prompts[0], [len(prompts[0]) - 1])])
    step.run_and_sample([StepEntry("s", None, [0])])
    before = step.buffers.h2d_bytes
    for _ in range(6):
        step.run_and_sample([StepEntry("s", None, [0])])
    assert step.buffers.h2d_bytes - before <= 6 * 4 * (2 + 2)     # at most a (count, count, index, page) a step
    step.free("s")


def test_records_outlive_preemption_at_the_step_function():
    """A request that is restarted (its pages given back, as the scheduler does on preemption)
    keeps its slot and its record: after recomputing prompt and generated tokens it goes on with
    the same generator counter, so its tokens are those of an undisturbed run."""
    from tokamak_b200.engine.replay import build_core
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    cfg, _, page = tiny_configs.ALL["B"][:3]
    core = build_core(model_folder("B", "float32"), "float32", max_tokens=256, page_size=page)
    step = core.step
    prompt = random_tokens(cfg["vocab_size"], 13, seed=3)
    row = SamplingRow(0.9, 30, 0.95, seed=77)

    def run(rid, restart_at=None):
        step.admit(rid, row)
        toks = step.run_and_sample([StepEntry(rid, prompt, [len(prompt) - 1])])
        for k in range(1, 14):
            if k == restart_at:
                slot = core.manager.slot(rid)
                step.restart(rid)
                assert core.manager.slot(rid) == slot and step.length(rid) == 0
                assert all(g.num_free == g.num_pages for g in core.manager.kv_groups)
                # everything so far is recomputed in two portions; the second samples the next token
                known = prompt + toks
                step.run([StepEntry(rid, known[:7], [])])
                toks += step.run_and_sample([StepEntry(rid, known[7:], [len(known) - 8])])
            else:
                toks += step.run_and_sample([StepEntry(rid, None, [0])])
        assert step.record(rid)["counter"] == len(toks) == 14
        step.free(rid)
        return toks

    assert run("calm") == run("shaken", restart_at=6)


def test_pool_sized_from_free_memory():
    """kv_pool_tokens="auto": the pool fills a share of the free device memory after a probe
    step has measured what a step needs, holds whole pages, never less than one request's
    maximum, and generation is what it is with the default pool."""
    from tokamak_b200 import SamplingParams
    prompts = prompts_for("A", [9, 21])
    params = SamplingParams(temperature=0.0, max_new_tokens=6)
    want = [o.output_token_ids for o in llm_for("A", "float32").generate(prompt_token_ids=prompts,
                                                                         sampling_params=params)]
    free, _ = torch.cuda.mem_get_info()
    share = 256e6 / free                                     # about 256 MB of pages
    llm = llm_for("A", "float32", kv_pool_tokens="auto", gpu_memory_utilization=share, max_seq_len=128)
    group = llm.cache_manager.kv_groups[0]
    per_token = llm.core.cache.bytes_per_token()
    assert group.num_pages * group.page_size >= 128
    assert 0.5 * 256e6 < group.num_pages * group.page_size * per_token <= 256e6
    assert [o.output_token_ids for o in llm.generate(prompt_token_ids=prompts, sampling_params=params)] == want
    tiny = llm_for("A", "float32", kv_pool_tokens="auto", gpu_memory_utilization=1e-9, max_seq_len=128)
    assert tiny.cache_manager.kv_groups[0].num_pages * tiny.cache_manager.kv_groups[0].page_size >= 128
    with pytest.raises(ValueError, match="'auto'"):
        llm_for("A", "float32", kv_pool_tokens="most")
