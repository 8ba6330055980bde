"""The reference arm of ``bench.py``: WeichunK/tokamak itself, unmodified, on the same metric.

The reference is installed into ``baseline/_ref`` (the folder is not part of the
history).  This module prepares what the reference needs as *input* and then goes
through its public API only, ``tokamak.LLM(folder).generate(prompt_token_ids=...,
sampling_params=SamplingParams(...))`` (src/tokamak/engine/llm.py:64-122, 265-286),
with its stock code path: its own model code, its paged cache, its scheduler and its
decode attention kernel.  Nothing of ``tokamak_b200`` is imported here.

Input that is prepared:
  * a model folder of seeded random bfloat16 weights under the checkpoint names the
    reference binds by (src/tokamak/model/loader.py:57-94), written shard by shard;
  * a stand-in tokenizer (``tokenizer.json`` with a handful of words): the reference's
    constructor loads one from the folder (llm.py:143) although the measurement passes
    token ids and never encodes or decodes text.

How the metric is read.  ``generate`` is called with B prompts of equal length and
``max_new_tokens = K + 1``, greedy, ``ignore_eos``.  The reference computes the B prompts one
after the other and only then decodes all B sequences together (scheduler.py:105-137), so the
K decode steps lie between the last request's first token and the end:
``max(latency_s) - max(ttft_s)``, both taken by the reference itself after the tokens have
reached the host (llm.py:447-460).  A first call with the same shapes warms everything up
(kernel compilation, library handles) and is not timed.
"""

from __future__ import annotations

import json
import shutil
import statistics
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REF_DIR = ROOT / "_ref"


def available() -> str | None:
    """``None`` when the installed reference is there, else the reason in one line."""
    if not (REF_DIR / "tokamak" / "__init__.py").is_file():
        return ("WeichunK/tokamak is not installed under baseline/_ref (pip install --no-index of it "
                "needs its build backend hatchling, which is neither installed nor in the wheelhouse)")
    return None


def _layer_names(i: int, cfg: dict) -> dict[str, tuple[int, ...]]:
    h, d = cfg["hidden_size"], cfg["head_dim"]
    hq, hkv, inter = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"]
    p = f"model.layers.{i}."
    return {
        p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
        p + "self_attn.q_proj.weight": (hq * d, h), p + "self_attn.k_proj.weight": (hkv * d, h),
        p + "self_attn.v_proj.weight": (hkv * d, h), p + "self_attn.o_proj.weight": (h, hq * d),
        p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
        p + "mlp.gate_proj.weight": (inter, h), p + "mlp.up_proj.weight": (inter, h),
        p + "mlp.down_proj.weight": (h, inter),
    }


def write_model_folder(folder: Path, cfg: dict, seed: int, device: str, std: float = 0.02) -> None:
    """config.json, one safetensors shard per layer, and the stand-in tokenizer."""
    import torch
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    raw = dict(cfg)
    raw.setdefault("model_type", "qwen3")
    raw.setdefault("torch_dtype", "bfloat16")
    raw.setdefault("hidden_act", "silu")
    (folder / "config.json").write_text(json.dumps(raw, indent=2))

    gen = torch.Generator(device=device).manual_seed(seed)

    def draw(shape):
        if len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
        else:
            t = std * torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
        return t.to(torch.bfloat16).cpu().contiguous()

    h, v = cfg["hidden_size"], cfg["vocab_size"]
    outer = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,)}
    if not cfg.get("tie_word_embeddings", False):
        outer["lm_head.weight"] = (v, h)
    n_layers = cfg["num_hidden_layers"]
    save_file({k: draw(s) for k, s in outer.items()}, str(folder / f"model-{0:05d}.safetensors"))
    for i in range(n_layers):
        save_file({k: draw(s) for k, s in _layer_names(i, cfg).items()},
                  str(folder / f"model-{i + 1:05d}.safetensors"))

    from tokenizers import Tokenizer, models, pre_tokenizers
    words = {"<unk>": 0, "<eos>": 1, "a": 2, "b": 3}
    tok = Tokenizer(models.WordLevel(words, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "eos_token": "<eos>"}))


def _scratch_folder(need_bytes: int) -> Path:
    """A temporary folder on a file system with room for the weights."""
    for base in (tempfile.gettempdir(), "/dev/shm"):
        try:
            if shutil.disk_usage(base).free > need_bytes * 1.1:
                return Path(tempfile.mkdtemp(prefix="tokamak_ref_model_", dir=base))
        except OSError:
            continue
    raise RuntimeError(f"no temporary folder with {need_bytes / 1e9:.1f} GB free for the reference's weights")


def _param_count(cfg: dict) -> int:
    per_layer = sum(s[0] * (s[1] if len(s) > 1 else 1) for s in _layer_names(0, cfg).values())
    outer = cfg["vocab_size"] * cfg["hidden_size"] * (1 if cfg.get("tie_word_embeddings") else 2)
    return per_layer * cfg["num_hidden_layers"] + outer + cfg["hidden_size"]


def _prompts(batch: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(batch)]


def _decode_run(llm, SamplingParams, batch: int, ctx: int, steps: int, vocab: int, seed: int) -> dict:
    """``steps`` decode steps of ``batch`` sequences whose context ends at ``ctx``."""
    params = SamplingParams(temperature=0.0, max_new_tokens=steps + 1, ignore_eos=True)
    prompt_len = ctx - steps - 1
    outs = llm.generate(prompt_token_ids=_prompts(batch, prompt_len, vocab, seed), sampling_params=params,
                        use_tqdm=False)
    if any(len(o.output_token_ids) != steps + 1 for o in outs):
        raise RuntimeError("the reference did not produce the asked number of tokens")
    seconds = max(o.latency_s for o in outs) - max(o.ttft_s for o in outs)
    return {"tok_s": batch * steps / seconds, "ms_per_step": seconds / steps * 1e3, "prompt_len": prompt_len}


def run(cfg: dict, model_name: str, batch: int, ctx: int, prefill_tokens: int, steps: int, warmup: int,
        points: tuple[int, ...] = (1, 64), device: str = "cuda", dtype: str = "bfloat16",
        clock_sampler=None, keep_folder: Path | None = None, config: dict | None = None) -> dict:
    """Measure the reference and return the bench line (``impl: reference``).  ``config`` is the
    record of sizes that the caller prints for the same run of its own arm."""
    sys.path.insert(0, str(REF_DIR))
    import torch
    from tokamak import LLM, SamplingParams

    vocab = cfg["vocab_size"]
    max_batch = max((batch,) + tuple(points))
    folder = keep_folder or _scratch_folder(_param_count(cfg) * 2)
    try:
        t0 = time.perf_counter()
        write_model_folder(folder, cfg, seed=0, device=device if device != "cpu" else "cpu")
        print(f"[reference arm] model folder written in {time.perf_counter() - t0:.0f}s", file=sys.stderr, flush=True)
        t0 = time.perf_counter()
        llm = LLM(str(folder), device=device, dtype=dtype, max_seq_len=max(ctx, prefill_tokens + 1),
                  block_size=16, kv_pool_tokens=max_batch * ctx, max_batch_size=max_batch)
        print(f"[reference arm] loaded in {time.perf_counter() - t0:.0f}s, attention backend "
              f"{llm.attention_backend}", file=sys.stderr, flush=True)
    finally:
        if keep_folder is None:
            shutil.rmtree(folder, ignore_errors=True)

    # untimed: the same shapes once, with at least three decode steps
    _decode_run(llm, SamplingParams, batch, ctx, max(3, warmup), vocab, seed=1)
    if clock_sampler is not None:
        clock_sampler.start()
    main = _decode_run(llm, SamplingParams, batch, ctx, steps, vocab, seed=2)

    # one prompt of `prefill_tokens` tokens to its first token (the warm-up above has compiled everything
    # but this length's library kernels: one untimed call first)
    one = SamplingParams(temperature=0.0, max_new_tokens=1, ignore_eos=True)
    times = []
    for i in range(4):
        out = llm.generate(prompt_token_ids=_prompts(1, prefill_tokens, vocab, 10 + i), sampling_params=one,
                           use_tqdm=False)[0]
        if i:
            times.append(out.ttft_s)
    prefill_s = statistics.median(times)

    pts = {}
    for b in points:
        _decode_run(llm, SamplingParams, b, ctx, 3, vocab, seed=20 + b)
        pts[f"decode_b{b}"] = round(_decode_run(llm, SamplingParams, b, ctx, steps, vocab, seed=30 + b)["tok_s"], 1)
    clocks = clock_sampler.stop() if clock_sampler is not None else None
    if device != "cpu":
        torch.cuda.synchronize()

    line = {
        "impl": "reference",
        "metric": f"decode tok/s at batch {batch} ({model_name} layer sizes, context {ctx})",
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": max(3, warmup), "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dtype == "bfloat16" else dtype,
        "data": "synthetic: seeded random weights N(0, 0.02), uniform random token ids",
        "config": dict(config) if config is not None else {
            "model": f"{model_name} layer sizes", "layers": cfg["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": vocab, "global_batch": batch, "seq_len": ctx,
            "prefill_tokens": prefill_tokens, "kv_block": 16, "parallelism": "single GPU",
        },
        "prompt_tokens": main["prompt_len"],
        "attention_backend": str(llm.attention_backend),
        "timing": "the reference's own timestamps around its decode steps (tokens on the host)",
        # the reference has one way in and out: token ids from the host, sampled tokens read back every step
        "e2e": {"value": round(main["tok_s"], 2), "unit": "tokens/s", "ms_per_step": round(main["ms_per_step"], 2)},
        "prefill": {"value": round(prefill_tokens / prefill_s, 1), "tokens": prefill_tokens,
                    "ms": round(prefill_s * 1e3, 3)},
        "points": pts,
    }
    if clocks is not None:
        line["clocks"] = clocks
    return line
