"""Live checks against WeichunK/tokamak's own code, where it can be imported.

The always-on oracle of these tests is the plain implementation under ``tests/plain``; the
committed golden logits pin it to the reference's model code.  Where the reference's package
is at hand (installed under ``baseline/_ref``, a source tree named by the environment variable
``TOKAMAK_REFERENCE_SRC``, or a ``reference/src`` folder beside the repository), three more
checks run; otherwise they skip:

* the golden logits are made again, in this process, by the reference's model code and must
  equal the committed files;
* greedy tokens of tiny configuration A through this engine's ``LLM.generate`` equal those of
  the reference's own ``tokamak.LLM(...).generate`` (src/tokamak/engine/llm.py:265-334);
* this scheduler's decisions equal the reference ``Scheduler``'s
  (src/tokamak/engine/scheduler.py:105-188), driven by hand as the reference's own tests do
  (tests/unit/test_scheduler.py:105-132), on the workloads both can express: whole prompts, no
  portions.
"""

from __future__ import annotations

import importlib
import json
import os
import random
import sys
from pathlib import Path

import pytest
import torch
from safetensors import safe_open

import tiny_configs
from helpers import model_folder, random_tokens

ROOT = Path(__file__).resolve().parent.parent


def _reference():
    """The reference's package, imported from wherever it is at hand; skips the test if nowhere."""
    candidates = [os.environ.get("TOKAMAK_REFERENCE_SRC"), ROOT / "baseline" / "_ref",
                  ROOT.parent / "reference" / "src"]
    for cand in candidates:
        if cand and (Path(cand) / "tokamak" / "__init__.py").is_file():
            if str(cand) not in sys.path:
                sys.path.insert(0, str(cand))
            try:
                return importlib.import_module("tokamak")
            except Exception as exc:          # a dependency of the reference is missing here
                pytest.skip(f"the reference is at {cand} but does not import: {exc}")
    pytest.skip("WeichunK/tokamak is not at hand (baseline/_ref, TOKAMAK_REFERENCE_SRC, ../reference/src)")


@pytest.mark.parametrize("tag", ["A", "B"])
def test_golden_logits_are_what_the_reference_computes_now(tag):
    _reference()
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import make_golden
    logits, ids, digest = make_golden.reference_logits(tag)
    with safe_open(str(ROOT / "tests" / "golden" / f"tiny_{tag}.safetensors"), framework="pt") as f:
        assert f.metadata()["weights_sha256"] == digest
        assert f.get_tensor("token_ids").tolist() == ids
        # the same code on the same kind of machine; thread counts may reorder a sum
        torch.testing.assert_close(logits, f.get_tensor("logits"), rtol=1e-5, atol=1e-5)


def _with_stand_in_tokenizer(folder: Path, dest: Path) -> Path:
    """A copy of a model folder with what the reference's constructor loads beside the weights: a
    tokenizer (never used: token ids go in and come out) and the keys its config reader wants."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    dest.mkdir(parents=True, exist_ok=True)
    raw = json.loads((folder / "config.json").read_text())
    raw.setdefault("model_type", "qwen3")
    raw.setdefault("hidden_act", "silu")
    (dest / "config.json").write_text(json.dumps(raw))
    (dest / "model.safetensors").write_bytes((folder / "model.safetensors").read_bytes())
    tok = Tokenizer(models.WordLevel({"<unk>": 0, "<eos>": 1, "a": 2}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(dest / "tokenizer.json"))
    (dest / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "eos_token": "<eos>"}))
    return dest


@pytest.mark.gpu
@pytest.mark.parametrize("tag,lengths,new", [("A", (5, 17, 33), 8), ("B", (1, 7, 31, 64), 12)])
def test_greedy_tokens_equal_the_reference_engine(tmp_path, tag, lengths, new):
    """Greedy tokens in float32 through the reference's engine on the CPU and through this
    engine on the GPU: configuration A's workload (prompts of 5, 17 and 33 tokens, 8 new tokens
    each) and prompts of configuration B, whose untied head makes the tokens vary."""
    ref = _reference()
    from tokamak_b200 import LLM, SamplingParams
    raw, _, page = tiny_configs.ALL[tag]
    folder = _with_stand_in_tokenizer(model_folder(tag, "float32"), tmp_path / tag)
    prompts = [random_tokens(raw["vocab_size"], n, seed=7 * n + 1) for n in lengths]
    theirs = ref.LLM(str(folder), device="cpu", dtype="float32", block_size=page).generate(
        prompt_token_ids=prompts, sampling_params=ref.SamplingParams(temperature=0.0, max_new_tokens=new),
        use_tqdm=False)
    ours = LLM(model_folder(tag, "float32"), dtype="float32", block_size=page).generate(
        prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=new))
    for a, b in zip(ours, theirs):
        assert a.output_token_ids == list(b.output_token_ids)
        assert a.finish_reason.value == b.finish_reason.value


# ---- scheduler decisions -----------------------------------------------------------------------

def _events_of_reference(ref, prompts, max_new, num_pages, page, max_batch):
    sched_mod = importlib.import_module("tokamak.engine.scheduler")
    seq_mod = importlib.import_module("tokamak.engine.sequence")
    mem = importlib.import_module("tokamak.memory")
    manager = mem.BlockManager(num_pages, page)
    sched = sched_mod.Scheduler(manager, max_batch)
    seqs = [seq_mod.Sequence(i, prompt_token_ids=[1] * n, sampling_params=ref.SamplingParams(max_new_tokens=m))
            for i, (n, m) in enumerate(zip(prompts, max_new))]
    for s in seqs:
        sched.add(s)
    events, started = [], set()

    def sample(s):
        s.append_output_token(0)
        if s.num_output_tokens >= s.sampling_params.max_new_tokens:
            s.finish(seq_mod.FinishReason.LENGTH)
            manager.free(s.seq_id)
            events.append(("finish", s.seq_id, s.num_tokens))

    while sched.has_unfinished():
        batch = sched.schedule()
        events += [("preempt", v.seq_id, v.num_tokens) for v in batch.preempted]
        if batch.kind is sched_mod.StepKind.PREFILL:
            s = batch.seqs[0]
            events.append(("restart" if s.seq_id in started else "start", s.seq_id, s.num_tokens))
            started.add(s.seq_id)
            sample(s)
        else:
            events.append(("decode", tuple(s.seq_id for s in batch.seqs)))
            for s in batch.seqs:
                sample(s)
    return events


def _events_of_ours(prompts, max_new, num_pages, page, max_batch):
    from tokamak_b200 import SamplingParams
    from tokamak_b200.cache.manager import CacheManager, KVGroup, KVPagesNeed
    from tokamak_b200.engine.scheduler import Scheduler
    from tokamak_b200.engine.sequence import Sequence
    manager = CacheManager([KVGroup(KVPagesNeed(1, 16), num_pages, page, ["kv"])], [], max_batch)
    sched = Scheduler(manager, max_batch, max_num_batched_tokens=10 ** 6)          # whole prompts only
    seqs = [Sequence(i, [1] * n, SamplingParams(max_new_tokens=m)) for i, (n, m) in enumerate(zip(prompts, max_new))]
    for s in seqs:
        sched.add(s)
    events, started = [], set()
    while sched.has_unfinished():
        plan = sched.schedule()
        events += [("preempt", v.seq_id, v.num_tokens) for v in plan.preempted]
        decoding = tuple(e.seq.seq_id for e in plan.entries if e.start > 0)
        for e in plan.entries:
            if e.start == 0:
                assert e.count == e.seq.num_tokens and e.samples            # a whole prompt, never a portion
                events.append(("restart" if e.seq.seq_id in started else "start", e.seq.seq_id, e.seq.num_tokens))
                started.add(e.seq.seq_id)
        if decoding:
            events.append(("decode", decoding))
        for e in plan.entries:
            manager.advance(e.seq.seq_id, e.count)
            e.seq.num_computed = e.start + e.count
            if e.seq.append_checked(0, eos_token_ids=(), max_total_tokens=10 ** 9):
                manager.free(e.seq.seq_id)
                events.append(("finish", e.seq.seq_id, e.seq.num_tokens))
    return events


def _comparable(events, n_requests):
    """The part of an event list on which the two schedulers must agree.

    Two differences are by design.  The reference computes one prompt per step while the running
    sequences stand still; this engine computes prompts in the same step as the running
    sequences' next tokens.  And when something waits, the reference asks first whether its
    prompt fits and then finds the pages for the running sequences' next tokens
    (scheduler.py:113-131), so it may admit a request that the next step evicts again; this
    scheduler serves the running sequences first and admits into what is left.  Both only
    matter once a decision about a waiting request is taken while others run.  Up to that moment
    the two are in the same state after the same events: the initial starts in arrival order
    under the slot and page gates, the decode steps in lockstep, and who is preempted first, and
    when.  The comparable part therefore ends with the first preemption, or with the first
    request that finishes while another one waits."""
    head, started = [], set()
    for ev in events:
        head.append(ev)
        if ev[0] == "start":
            started.add(ev[1])
        elif ev[0] == "preempt" or (ev[0] == "finish" and len(started) < n_requests):
            break
    return head


@pytest.mark.parametrize("seed", range(10))
def test_scheduler_decisions_equal_the_reference_scheduler(seed):
    ref = _reference()
    rng = random.Random(seed)
    page = rng.choice((2, 4, 8))
    max_batch = rng.randint(2, 5)
    n = rng.randint(max_batch, max_batch + 3)
    prompts = [rng.randint(1, 6 * page) for _ in range(n)]
    max_new = [rng.randint(2, 5 * page) for _ in range(n)]
    # a pool in which every request fits alone, tight enough that running sequences collide
    alone = max(-(-(p + m) // page) for p, m in zip(prompts, max_new))
    num_pages = alone + rng.randint(0, 2 * alone)
    theirs = _events_of_reference(ref, prompts, max_new, num_pages, page, max_batch)
    ours = _events_of_ours(prompts, max_new, num_pages, page, max_batch)
    assert _comparable(ours, n) == _comparable(theirs, n)
    # whatever the timing, both start the requests in arrival order and finish every one of them
    first_starts = lambda evs: [e[1] for e in evs if e[0] == "start"]
    assert first_starts(ours) == first_starts(theirs) == list(range(n))
    finished = lambda evs: sorted((e[1], e[2]) for e in evs if e[0] == "finish")
    assert finished(ours) == finished(theirs)


def test_scheduler_equals_the_reference_when_nothing_is_admitted_late():
    """Everything fits the batch from the start and the pool is tight: after the prompts both
    schedulers only decode until the pool runs out: the same sequence is preempted, at the same
    length, after the same number of decode steps."""
    ref = _reference()
    args = ([7, 7, 6, 5], [12, 12, 12, 12], 9, 4, 4)
    theirs, ours = _events_of_reference(ref, *args), _events_of_ours(*args)
    assert _comparable(ours, 4)[-1][0] == "preempt"
    assert _comparable(ours, 4) == _comparable(theirs, 4)
