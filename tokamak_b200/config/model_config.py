"""Typed configuration of the Qwen3 dense decoder, read from ``config.json`` keys.

Same fields and defaults as the reference's ``ModelConfig``
(``src/tokamak/config.py:29-126``), but parsed from the raw JSON dictionary so
that no third-party config object is needed.  Every size the model code uses
comes from here; nothing is hard-coded elsewhere.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Sequence


class ConfigError(ValueError):
    """A ``config.json`` that this engine cannot run."""


def _require(raw: Mapping[str, Any], key: str) -> Any:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json is missing required key {key!r}")
    return raw[key]


def resolve_rope_theta(raw: Mapping[str, Any]) -> float:
    """RoPE base across the two config layouts (``src/tokamak/config.py:129-157``).

    Layout 1: a ``rope_parameters`` dict whose ``rope_type`` must be ``default``.
    Layout 2: flat ``rope_theta`` with ``rope_scaling`` absent or null.
    A base that cannot be found is an error, never a silent default.
    """
    rope_parameters = raw.get("rope_parameters")
    if isinstance(rope_parameters, Mapping):
        rope_type = rope_parameters.get("rope_type", "default")
        if rope_type != "default":
            raise ConfigError(f"RoPE scaling type {rope_type!r} is not supported")
        theta = rope_parameters.get("rope_theta")
        if theta is not None:
            return float(theta)
    theta = raw.get("rope_theta")
    if theta is not None:
        rope_scaling = raw.get("rope_scaling")
        if rope_scaling is not None:
            raise ConfigError(f"RoPE scaling is not supported (got {rope_scaling!r})")
        return float(theta)
    raise ConfigError("Could not determine rope_theta from the model config")


@dataclass(frozen=True, slots=True)
class ModelConfig:
    """Hyperparameters of a dense GQA decoder (``src/tokamak/config.py:29-78``).

    ``sliding_window`` is ``None`` for full attention.  When set, layers with
    index ``>= max_window_layers`` see only the last ``sliding_window``
    positions (query included), the visibility rule of the reference's window
    policy (``src/tokamak/model/attention_policy.py:22-61``) applied per layer.
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    num_layers: int
    num_attention_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    use_qk_norm: bool = True
    eos_token_ids: tuple[int, ...] = ()
    sliding_window: int | None = None
    max_window_layers: int = 0

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "num_layers", "num_attention_heads",
                     "num_kv_heads", "head_dim", "intermediate_size", "max_position_embeddings"):
            if int(getattr(self, name)) < 1:
                raise ConfigError(f"{name} must be >= 1, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_kv_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible "
                f"by num_kv_heads ({self.num_kv_heads})"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotary embedding, got {self.head_dim}")
        if not self.rms_norm_eps > 0.0:
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if self.sliding_window is not None and self.sliding_window < 1:
            raise ConfigError(f"sliding_window must be >= 1, got {self.sliding_window}")

    @property
    def num_kv_groups(self) -> int:
        """Query heads per key/value head."""
        return self.num_attention_heads // self.num_kv_heads

    def layer_window(self, layer_idx: int) -> int | None:
        """Window of one layer, ``None`` for full attention."""
        if self.sliding_window is None or layer_idx < self.max_window_layers:
            return None
        return self.sliding_window

    @classmethod
    def from_json_dict(cls, raw: Mapping[str, Any], eos_token_ids: Sequence[int] | None = None,
                       *, qk_norm: bool = True, attention_bias_default: bool = False) -> "ModelConfig":
        """Build from the dictionary stored in ``config.json`` (``src/tokamak/config.py:80-126``)."""
        architectures = raw.get("architectures") or []
        architecture = architectures[0] if architectures else "<missing>"
        num_heads = int(_require(raw, "num_attention_heads"))
        hidden = int(_require(raw, "hidden_size"))
        head_dim = raw.get("head_dim")
        if head_dim is None:
            head_dim = hidden // num_heads
        num_kv = raw.get("num_key_value_heads")
        if num_kv is None:
            num_kv = num_heads
        if eos_token_ids is None:
            eos_raw = raw.get("eos_token_id")
            if isinstance(eos_raw, int):
                eos_token_ids = (eos_raw,)
            elif isinstance(eos_raw, (list, tuple)):
                eos_token_ids = tuple(int(e) for e in eos_raw)
            else:
                eos_token_ids = ()
        window = None
        if raw.get("use_sliding_window"):
            window = int(_require(raw, "sliding_window"))
        return cls(
            architecture=architecture,
            vocab_size=int(_require(raw, "vocab_size")),
            hidden_size=hidden,
            num_layers=int(_require(raw, "num_hidden_layers")),
            num_attention_heads=num_heads,
            num_kv_heads=int(num_kv),
            head_dim=int(head_dim),
            intermediate_size=int(_require(raw, "intermediate_size")),
            rms_norm_eps=float(_require(raw, "rms_norm_eps")),
            rope_theta=resolve_rope_theta(raw),
            max_position_embeddings=int(_require(raw, "max_position_embeddings")),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", attention_bias_default)),
            use_qk_norm=qk_norm,
            eos_token_ids=tuple(int(e) for e in eos_token_ids),
            sliding_window=window,
            max_window_layers=int(raw.get("max_window_layers") or 0) if window is not None else 0,
        )

    def to_json_dict(self) -> dict[str, Any]:
        """The ``config.json`` dictionary that parses back to this configuration."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "hidden_act": "silu",
            "use_sliding_window": self.sliding_window is not None,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    """Load ``config.json`` of a model folder as a dictionary."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"No config.json under {model_dir}")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return raw


def read_eos_token_ids(model_dir: str | Path, raw_config: Mapping[str, Any]) -> tuple[int, ...]:
    """EOS ids: ``generation_config.json`` first, then ``config.json``.

    The reference resolves them from the generation config before falling back
    (``src/tokamak/engine/llm.py:244-263``); a folder of random weights has
    neither file nor key and then generation stops only on length.
    """
    gen_path = Path(model_dir) / "generation_config.json"
    raw: Any = None
    if gen_path.is_file():
        with open(gen_path, "r", encoding="utf-8") as f:
            raw = json.load(f).get("eos_token_id")
    if raw is None:
        raw = raw_config.get("eos_token_id")
    if isinstance(raw, int):
        return (raw,)
    if isinstance(raw, (list, tuple)):
        return tuple(int(e) for e in raw)
    return ()
