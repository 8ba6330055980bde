"""Configuration parsing and the architecture registry (after the reference's
tests/unit/test_config.py)."""

from __future__ import annotations

import copy
import json

import pytest

import tiny_configs
from tokamak_b200.config import (ConfigError, ModelConfig, architecture_of, read_config_json,
                                 read_eos_token_ids, supported_architectures)


def test_tiny_configs_parse_and_differ_everywhere():
    a = architecture_of(tiny_configs.TINY_A).parse_config(tiny_configs.TINY_A)
    b = architecture_of(tiny_configs.TINY_B).parse_config(tiny_configs.TINY_B)
    assert a.architecture == b.architecture == "Qwen3ForCausalLM"
    for field in ("vocab_size", "hidden_size", "num_layers", "num_attention_heads", "num_kv_heads",
                  "head_dim", "intermediate_size", "rms_norm_eps", "rope_theta",
                  "max_position_embeddings", "tie_word_embeddings", "num_kv_groups"):
        assert getattr(a, field) != getattr(b, field), field
    assert b.num_attention_heads * b.head_dim != b.hidden_size
    assert a.use_qk_norm and b.use_qk_norm and not a.attention_bias


def test_both_rope_layouts_and_errors():
    raw = copy.deepcopy(tiny_configs.TINY_A)
    assert ModelConfig.from_json_dict(raw).rope_theta == 10000.0
    raw2 = copy.deepcopy(tiny_configs.TINY_B)
    assert ModelConfig.from_json_dict(raw2).rope_theta == 1e6
    raw["rope_scaling"] = {"type": "linear", "factor": 2.0}
    with pytest.raises(ConfigError, match="RoPE scaling"):
        ModelConfig.from_json_dict(raw)
    raw["rope_scaling"] = None
    ModelConfig.from_json_dict(raw)
    raw2["rope_parameters"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError, match="yarn"):
        ModelConfig.from_json_dict(raw2)
    del raw["rope_theta"]
    with pytest.raises(ConfigError, match="rope_theta"):
        ModelConfig.from_json_dict(raw)


def test_defaults_and_validation():
    raw = copy.deepcopy(tiny_configs.TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"], raw["tie_word_embeddings"]
    cfg = ModelConfig.from_json_dict(raw)
    assert cfg.head_dim == 16 and cfg.num_kv_heads == 4 and cfg.tie_word_embeddings is False
    raw["num_key_value_heads"] = 3
    with pytest.raises(ConfigError, match="divisible"):
        ModelConfig.from_json_dict(raw)
    raw["num_key_value_heads"] = 2
    raw["head_dim"] = 15
    with pytest.raises(ConfigError, match="even"):
        ModelConfig.from_json_dict(raw)
    raw["head_dim"] = 16
    del raw["vocab_size"]
    with pytest.raises(ConfigError, match="vocab_size"):
        ModelConfig.from_json_dict(raw)


def test_ignored_keys_and_window():
    raw = copy.deepcopy(tiny_configs.TINY_A)
    raw.update(hidden_act="silu", attention_dropout=0.0, initializer_range=0.02, torch_dtype="bfloat16",
               bos_token_id=1, sliding_window=4096, use_sliding_window=False, max_window_layers=28)
    cfg = ModelConfig.from_json_dict(raw)
    assert cfg.sliding_window is None and cfg.layer_window(1) is None
    w = ModelConfig.from_json_dict(tiny_configs.TINY_W)
    assert [w.layer_window(i) for i in range(3)] == [None, 24, 24]
    assert ModelConfig.from_json_dict(w.to_json_dict()) == w


def test_registry_errors():
    assert supported_architectures() == ["Qwen3ForCausalLM"]
    with pytest.raises(ConfigError, match="Unsupported architecture 'LlamaForCausalLM'; supported: Qwen3"):
        architecture_of({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="<missing>"):
        architecture_of({})
    raw = copy.deepcopy(tiny_configs.TINY_A)
    raw["attention_bias"] = True
    with pytest.raises(ConfigError, match="attention_bias"):
        architecture_of(raw).parse_config(raw)


def test_eos_ids_from_files(tmp_path):
    raw = copy.deepcopy(tiny_configs.TINY_A)
    raw["eos_token_id"] = 7
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert read_eos_token_ids(tmp_path, read_config_json(tmp_path)) == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 9]}))
    assert read_eos_token_ids(tmp_path, read_config_json(tmp_path)) == (3, 9)
    with pytest.raises(FileNotFoundError):
        read_config_json(tmp_path / "nowhere")


def test_model_spec_is_data():
    from tokamak_b200.models import qwen3
    cfg = qwen3.parse_config(tiny_configs.TINY_W)
    spec = qwen3.model_spec(cfg)
    assert [c.block for c in spec.schedule] == ["layers.0", "layers.1", "layers.2"]
    assert [b.mixer.window for b in spec.blocks] == [None, 24, 24]
    assert spec.blocks[0].mixer.position.theta == 50000.0
    assert spec.blocks[0].mixer.qk_norm_eps == cfg.rms_norm_eps


def test_the_engine_protocol_of_a_configuration_is_checked_and_options_are_refused_by_name():
    """What the engine reads from a typed configuration is a written protocol that every parsed
    configuration is checked against; engine-wide options reach ``model_spec`` as arguments, and an
    architecture that does not list one refuses it with the reason."""
    from dataclasses import dataclass
    from tokamak_b200.config import (Architecture, ConfigError, architecture_of, register_architecture,
                                     unregister_architecture)

    @dataclass(frozen=True)
    class Good:
        vocab_size: int = 10
        max_position_embeddings: int = 32
        eos_token_ids: tuple = ()
        architecture: str = "ToyProtocol"

    @dataclass(frozen=True)
    class Bad:
        vocab_size: float = 10.0
        eos_token_ids: tuple = ()
        architecture: str = "ToyProtocol"

    seen = {}

    def model_spec(cfg, **options):
        seen.update(options)
        return "spec"

    try:
        register_architecture(Architecture("ToyProtocol", lambda raw, eos=None: Good(), model_spec))
        arch = architecture_of({"architectures": ["ToyProtocol"]})
        cfg = arch.parse({})
        assert arch.build_spec(cfg, window=None) == "spec" and seen == {}
        with pytest.raises(ConfigError, match="does not take the engine option 'window'"):
            arch.build_spec(cfg, window=16)
        register_architecture(Architecture("ToyProtocol", lambda raw, eos=None: Good(), model_spec,
                                           options=frozenset({"window"})))
        assert architecture_of({"architectures": ["ToyProtocol"]}).build_spec(cfg, window=16) == "spec"
        assert seen == {"window": 16}
        register_architecture(Architecture("ToyProtocol", lambda raw, eos=None: Bad(), model_spec))
        with pytest.raises(ConfigError, match="max_position_embeddings is missing") as info:
            architecture_of({"architectures": ["ToyProtocol"]}).parse({})
        assert "vocab_size must be int" in str(info.value)
        with pytest.raises(ConfigError, match="options that do not exist"):
            register_architecture(Architecture("ToyProtocol", Good, model_spec, options=frozenset({"turbo"})))
        with pytest.raises(ConfigError, match="callable"):
            register_architecture(Architecture("ToyProtocol", None, model_spec))
    finally:
        unregister_architecture("ToyProtocol")
    # the built-in architecture takes the window as an argument and windows every layer with it
    from tokamak_b200.models import qwen3
    import tiny_configs
    qcfg = architecture_of(tiny_configs.TINY_A).parse(tiny_configs.TINY_A)
    spec = architecture_of(tiny_configs.TINY_A).build_spec(qcfg, window=12)
    assert all(b.mixer.window == 12 for b in spec.blocks)
    assert all(b.mixer.window is None for b in qwen3.model_spec(qcfg).blocks)
