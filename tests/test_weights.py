"""Weight loading: coverage errors in one message, dtypes in memory, the random writer."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny_configs
from helpers import model_folder
from tokamak_b200.config import architecture_of
from tokamak_b200.models.decoder import DecoderModel
from tokamak_b200.weights import WeightsError, load_tensors, write_random_model


def expected_for(raw):
    arch = architecture_of(raw)
    return DecoderModel.expected_tensors(arch.model_spec(arch.parse_config(raw)))


def test_expected_names_match_the_checkpoint_layout():
    exp = expected_for(tiny_configs.TINY_A)
    L = tiny_configs.TINY_A["num_hidden_layers"]
    required = [n for n, r in exp.items() if not r.optional]
    assert len(required) == 11 * L + 2                       # tied: the head is optional
    assert "model.layers.1.self_attn.q_norm.weight" in exp and "model.norm.weight" in exp
    expB = expected_for(tiny_configs.TINY_B)
    assert not expB["lm_head.weight"].optional
    assert expB["model.layers.0.self_attn.q_proj.weight"].shape == (192, 96)
    assert expB["model.layers.2.mlp.down_proj.weight"].shape == (96, 160)


def test_random_folder_is_reproducible_and_loads(tmp_path):
    a = write_random_model(tmp_path / "a", tiny_configs.TINY_B, seed=5, std=0.05, dtype="bfloat16")
    b = write_random_model(tmp_path / "b", tiny_configs.TINY_B, seed=5, std=0.05, dtype="bfloat16")
    c = write_random_model(tmp_path / "c", tiny_configs.TINY_B, seed=6, std=0.05, dtype="bfloat16")
    ta, tb, tc = (load_file(str(p / "model.safetensors")) for p in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    assert json.loads((a / "config.json").read_text())["vocab_size"] == 317
    w = ta["model.layers.0.mlp.up_proj.weight"].float()
    assert 0.04 < w.std() < 0.06 and abs(w.mean()) < 0.01
    n = ta["model.norm.weight"].float()
    assert 0.9 < n.mean() < 1.1 and 0.05 < n.std() < 0.15
    tensors = load_tensors(a, expected_for(tiny_configs.TINY_B), torch.bfloat16, "cpu")
    assert tensors["lm_head.weight"].dtype == torch.bfloat16
    assert tensors["model.norm.weight"].dtype == torch.float32          # per-channel vectors stay 32-bit
    t32 = load_tensors(a, expected_for(tiny_configs.TINY_B), torch.float32, "cpu")
    assert t32["lm_head.weight"].dtype == torch.float32
    assert torch.equal(t32["lm_head.weight"], ta["lm_head.weight"].float())


def test_one_error_lists_every_fault(tmp_path):
    folder = write_random_model(tmp_path / "m", tiny_configs.TINY_B, seed=1, dtype="float32")
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(31)
    tensors["model.embed_tokens.weight"] = torch.zeros(317, 95)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightsError) as info:
        load_tensors(folder, expected_for(tiny_configs.TINY_B), torch.float32, "cpu")
    err = info.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert [w[0] for w in err.wrong_shape] == ["model.embed_tokens.weight",
                                              "model.layers.2.self_attn.k_norm.weight"]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "(317, 95)", "(317, 96)"):
        assert needle in text


def test_tied_head_is_optional_and_no_files_is_an_error(tmp_path):
    folder = write_random_model(tmp_path / "m", tiny_configs.TINY_A, seed=0, dtype="float32")
    tensors = load_file(str(folder / "model.safetensors"))
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(folder / "model.safetensors"))
    load_tensors(folder, expected_for(tiny_configs.TINY_A), torch.float32, "cpu")   # stray head is fine
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        load_tensors(tmp_path / "empty", expected_for(tiny_configs.TINY_A), torch.float32, "cpu")
