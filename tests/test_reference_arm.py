"""The input that bench.py's reference arm prepares: a sharded folder under the checkpoint names.

The arm itself runs the reference's package, which is not part of the history; what can be
checked without it is that the folder it writes is a complete checkpoint of the named sizes:
this engine's own loader, which lists every missing, unexpected or misshapen tensor, accepts it.
"""

from __future__ import annotations

import importlib.util
import json
from pathlib import Path

import torch

import tiny_configs
from tokamak_b200.config import architecture_of
from tokamak_b200.models.decoder import DecoderModel
from tokamak_b200.weights import load_tensors

ARM = Path(__file__).resolve().parent.parent / "baseline" / "reference_arm.py"


def load_arm():
    spec = importlib.util.spec_from_file_location("reference_arm", ARM)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_folder_of_the_reference_arm_is_a_complete_checkpoint(tmp_path):
    arm = load_arm()
    for raw in (tiny_configs.TINY_A, tiny_configs.TINY_B):
        folder = tmp_path / raw["_name"] if "_name" in raw else tmp_path / str(raw["hidden_size"])
        arm.write_model_folder(folder, raw, seed=0, device="cpu")
        written = json.loads((folder / "config.json").read_text())
        arch = architecture_of(written)
        expected = DecoderModel.expected_tensors(arch.model_spec(arch.parse_config(written)))
        shards = sorted(folder.glob("*.safetensors"))
        assert len(shards) == raw["num_hidden_layers"] + 1
        tensors = load_tensors(folder, expected, torch.float32, "cpu")
        n_params = sum(t.numel() for n, t in tensors.items())
        assert n_params == arm._param_count(raw)
        assert (folder / "tokenizer.json").is_file()


def test_unavailable_says_why(tmp_path, monkeypatch):
    arm = load_arm()
    monkeypatch.setattr(arm, "REF_DIR", tmp_path / "nothing_here")
    why = arm.available()
    assert why is not None and "hatchling" in why
