"""The command line: the reference's option names and defaults, and the random-weights writer."""

from __future__ import annotations

import json

import tiny_configs
from tokamak_b200.cli import build_parser, main


def test_options_follow_the_reference_example():
    # examples/basic_generation.py:14-20 of the reference: --model --prompt --max-new-tokens 256
    # --temperature 0.7 --top-p 0.95
    args = build_parser().parse_args(["--model", "m"])
    assert (args.max_new_tokens, args.temperature, args.top_p) == (256, 0.7, 0.95)
    assert args.prompt == "What does an LLM inference engine do?"
    assert (args.block_size, args.max_batch_size, args.dtype, args.attention_policy) == (16, 16, "auto", "full")
    args = build_parser().parse_args(["--model", "m", "--prompt-token-ids", "1,2,3", "--temperature", "0",
                                      "--top-k", "5", "--seed", "9", "--prefill-chunk", "24"])
    assert args.prompt_token_ids == "1,2,3" and args.top_k == 5 and args.seed == 9 and args.prefill_chunk == 24


def test_write_random_from_the_command_line(tmp_path, capsys):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(tiny_configs.TINY_A))
    out = tmp_path / "model"
    assert main(["--write-random", str(out), "--config", str(cfg), "--seed", "3", "--weights-dtype", "float32"]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    assert "wrote" in capsys.readouterr().out
