"""Command line: generate from a model folder, or write a folder of random weights.

    python -m tokamak_b200.cli --model DIR --prompt "..." --max-new-tokens 256 \\
        --temperature 0.7 --top-p 0.95
    python -m tokamak_b200.cli --model DIR --prompt-token-ids 5,17,3 --temperature 0
    python -m tokamak_b200.cli --write-random DIR --config config.json --seed 0

``--model``, ``--prompt``, ``--max-new-tokens``, ``--temperature`` and ``--top-p`` are the
options of the reference's example (examples/basic_generation.py:14-20) with its defaults.
A folder of random weights has no tokenizer, so prompts can also be given as token ids
or as a length of seeded random ids.
"""

from __future__ import annotations

import argparse
import json
import sys


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--model", help="model folder (config.json + safetensors)")
    ap.add_argument("--prompt", default="What does an LLM inference engine do?")
    ap.add_argument("--prompt-token-ids", help="comma-separated token ids instead of --prompt")
    ap.add_argument("--prompt-len", type=int, help="use this many seeded random token ids as the prompt")
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=None, help="sampling seed (and seed of --write-random)")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--dtype", default="auto", choices=["auto", "bfloat16", "float32"])
    ap.add_argument("--max-seq-len", type=int, default=None)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--kv-pool-tokens", type=lambda v: v if v == "auto" else int(v), default=None,
                    help="tokens the page pool holds (default: max-seq-len), or 'auto' to fill the free memory")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--max-batch-size", type=int, default=16)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=None)
    ap.add_argument("--attention-policy", default="full")
    ap.add_argument("--kv-watermark", type=float, default=0.0,
                    help="share of the page pool that an admission leaves free while other requests run")
    ap.add_argument("--step-token-multiple", type=int, default=128,
                    help="a step of more tokens than this is cut down to a multiple of it by ending a prompt "
                         "portion earlier (the token tile of the matrix products; 1: steps as planned)")
    ap.add_argument("--write-random", metavar="DIR", help="write config.json and model.safetensors "
                    "with seeded random weights to DIR and exit")
    ap.add_argument("--config", help="config.json to take the sizes from (with --write-random)")
    ap.add_argument("--std", type=float, default=0.02)
    ap.add_argument("--weights-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    return ap


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if args.write_random:
        if not args.config:
            raise SystemExit("--write-random needs --config")
        from .weights import write_random_model
        with open(args.config, "r", encoding="utf-8") as f:
            raw = json.load(f)
        out = write_random_model(args.write_random, raw, seed=args.seed or 0, std=args.std,
                                 dtype=args.weights_dtype)
        print(f"wrote {out}")
        return 0
    if not args.model:
        raise SystemExit("--model is required")

    from . import LLM, SamplingParams

    llm = LLM(args.model, dtype=args.dtype, max_seq_len=args.max_seq_len, block_size=args.block_size,
              kv_pool_tokens=args.kv_pool_tokens, max_batch_size=args.max_batch_size,
              gpu_memory_utilization=args.gpu_memory_utilization,
              max_num_batched_tokens=args.max_num_batched_tokens, prefill_chunk=args.prefill_chunk,
              attention_policy=args.attention_policy, kv_watermark=args.kv_watermark,
              step_token_multiple=args.step_token_multiple)
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                            max_new_tokens=args.max_new_tokens, seed=args.seed,
                            ignore_eos=args.ignore_eos)
    if args.prompt_token_ids or args.prompt_len:
        if args.prompt_token_ids:
            ids = [int(t) for t in args.prompt_token_ids.split(",") if t.strip()]
        else:
            import torch
            gen = torch.Generator().manual_seed(args.seed or 0)
            ids = torch.randint(0, llm.model_config.vocab_size, (args.prompt_len,), generator=gen).tolist()
        outputs = llm.generate(prompt_token_ids=[ids], sampling_params=params)
        shown = f"{len(ids)} token ids"
    else:
        tok = llm.tokenizer
        # chat formatting is the tokenizer's job (examples/basic_generation.py:48-54)
        try:
            text = tok.apply_chat_template([{"role": "user", "content": args.prompt}], tokenize=False,
                                           add_generation_prompt=True, enable_thinking=False)
        except Exception:
            text = args.prompt
        outputs = llm.generate(text, params)
        shown = args.prompt
    out = outputs[0]
    print(f"\n[prompt]\n{shown}\n")
    print(f"[completion ({out.finish_reason.value})]")
    print(out.output_text if out.output_text else " ".join(str(t) for t in out.output_token_ids))
    return 0


if __name__ == "__main__":
    sys.exit(main())
