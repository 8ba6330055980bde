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


def test_llm_accepts_the_reference_options_at_their_defaults_and_refuses_the_rest():
    """A call written for the reference (src/tokamak/engine/llm.py:64-122) still works: the options
    that name parts this engine does not have are taken at their defaults and refused otherwise.
    The checks come before anything touches the device, so they run without one."""
    import types

    import pytest

    from tokamak_b200.engine.llm import LLM

    for bad in ({"kv_backend": "contiguous"}, {"scheduling": "static"}, {"attention_backend": "sdpa"},
                {"draft_model": "some/folder"}, {"attention_policy": "streaming:64+4"}, {"block_size": 0},
                {"max_batch_size": 0}):
        with pytest.raises(ValueError):
            LLM("nowhere", **bad)
    core = types.SimpleNamespace(config=None, max_seq_len=64, device="cuda:0", dtype=None, manager=None, model=None)
    llm = LLM("nowhere", kv_backend="paged", scheduling="continuous", attention_backend="auto", draft_model=None,
              num_speculative_tokens=4, _core=core)
    assert llm.max_seq_len == 64 and llm.max_batch_size == 16
