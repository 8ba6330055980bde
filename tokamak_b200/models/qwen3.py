"""The Qwen3 dense decoder as a :class:`ModelSpec`.

Grouped-query attention with per-head RMSNorm on q and k before the half
rotation, no biases, SwiGLU feed-forward, pre-norm residual blocks and a tied or
untied head, as src/tokamak/model/transformer.py runs it with
``use_qk_norm=True`` and ``attention_bias=False``.
"""

from __future__ import annotations

from typing import Any, Mapping

from ..config.model_config import ConfigError, ModelConfig
from ..parts.attention import AttentionSpec
from ..parts.block import PreNormBlockSpec
from ..parts.embedding import EmbeddingSpec, HeadSpec
from ..parts.feedforward import SwiGLUSpec
from ..parts.norm import RMSNormSpec
from ..parts.position import RopeSpec
from .decoder import LayerCall, ModelSpec

ARCHITECTURE = "Qwen3ForCausalLM"


def parse_config(raw: Mapping[str, Any], eos_token_ids=None) -> ModelConfig:
    """Read Qwen3's config.json keys; biases on q, k and v are not part of this architecture."""
    cfg = ModelConfig.from_json_dict(raw, eos_token_ids, qk_norm=True)
    if cfg.attention_bias:
        raise ConfigError("attention_bias=true is not supported for Qwen3ForCausalLM")
    return cfg


def model_spec(cfg: ModelConfig, window: int | None = None) -> ModelSpec:
    """Blocks and schedule of a configuration: every layer once, each with a cache of its own.

    ``window`` is the engine-wide option (``attention_policy="window:W"``): every layer sees
    the last ``W`` positions only, whatever the configuration says about windows."""
    blocks = []
    schedule = []
    for i in range(cfg.num_layers):
        prefix = f"model.layers.{i}."
        norm = RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps)
        mixer = AttentionSpec(
            hidden_size=cfg.hidden_size,
            num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_kv_heads,
            head_dim=cfg.head_dim,
            position=RopeSpec(cfg.head_dim, cfg.rope_theta),
            qk_norm_eps=cfg.rms_norm_eps if cfg.use_qk_norm else None,
            window=window if window is not None else cfg.layer_window(i),
        )
        blocks.append(PreNormBlockSpec(
            name=f"layers.{i}",
            norm1=norm, mixer=mixer, norm2=norm,
            feed_forward=SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size),
            norm1_name=prefix + "input_layernorm.weight",
            mixer_prefix=prefix + "self_attn.",
            norm2_name=prefix + "post_attention_layernorm.weight",
            ffn_prefix=prefix + "mlp.",
        ))
        schedule.append(LayerCall(block=f"layers.{i}", cache=f"layers.{i}"))
    return ModelSpec(
        embedding=EmbeddingSpec(cfg.vocab_size, cfg.hidden_size),
        blocks=tuple(blocks),
        schedule=tuple(schedule),
        final_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps),
        final_norm_name="model.norm.weight",
        head=HeadSpec(cfg.vocab_size, cfg.hidden_size, tied=cfg.tie_word_embeddings),
    )
