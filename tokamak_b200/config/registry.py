"""The one registry from an architecture's name to its model.

An architecture is two functions: ``parse_config`` turns the raw ``config.json``
dictionary into a typed configuration, and ``model_spec`` turns that into the
parts, blocks and schedule of the model.  Adding an architecture is adding an
entry (src/tokamak/config.py:20-26 is the reference's whitelist).

**What the engine reads from a typed configuration** is written down here and checked on
every configuration an architecture parses, so that another architecture's configuration can
be any object of its own making:

====================================  ======================================================
``vocab_size: int``                    token ids a request may bring; width of the logits
``max_position_embeddings: int``       upper bound of ``max_seq_len``
``eos_token_ids: tuple[int, ...]``     tokens that end a request (may be empty)
``architecture: str``                  the name it was registered under (for messages)
====================================  ======================================================

Everything else (sizes of layers, constants) is between ``parse_config`` and ``model_spec``.

**Engine-wide options** that change the model are arguments of ``model_spec``, not rewritten
configuration keys.  An architecture lists the ones it takes in ``options``; the engine refuses an
option that the architecture does not list, with the reason.  The one option so far is
``window`` (``attention_policy="window:W"``: every attention layer sees the last W positions).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .model_config import ConfigError

CONFIG_PROTOCOL = {"vocab_size": int, "max_position_embeddings": int, "eos_token_ids": tuple,
                   "architecture": str}
KNOWN_OPTIONS = frozenset({"window"})


def check_config_protocol(cfg: Any, name: str) -> Any:
    """Raise :class:`ConfigError` unless ``cfg`` has what the engine reads from a configuration."""
    faults = []
    for attr, kind in CONFIG_PROTOCOL.items():
        if not hasattr(cfg, attr):
            faults.append(f"{attr} is missing")
        elif not isinstance(getattr(cfg, attr), kind) or isinstance(getattr(cfg, attr), bool):
            faults.append(f"{attr} must be {kind.__name__}, got {type(getattr(cfg, attr)).__name__}")
    if not faults and (cfg.vocab_size < 1 or cfg.max_position_embeddings < 1):
        faults.append("vocab_size and max_position_embeddings must be positive")
    if faults:
        raise ConfigError(f"the configuration that architecture {name!r} parsed does not meet the "
                          f"engine's protocol: {'; '.join(faults)}")
    return cfg


@dataclass(frozen=True)
class Architecture:
    """``parse_config(raw, eos_token_ids) -> config``; ``model_spec(config, **options) -> ModelSpec``
    where ``options`` holds only names listed in ``options``."""

    name: str
    parse_config: Callable[..., Any]
    model_spec: Callable[..., Any]
    options: frozenset = frozenset()

    def parse(self, raw: Mapping[str, Any], eos_token_ids=None) -> Any:
        """The typed configuration, checked against the engine's protocol."""
        return check_config_protocol(self.parse_config(raw, eos_token_ids), self.name)

    def build_spec(self, cfg: Any, **options: Any) -> Any:
        """The model as data, with the engine-wide options that were asked for (``None`` = not asked)."""
        asked = {k: v for k, v in options.items() if v is not None}
        for key in asked:
            if key not in self.options:
                raise ConfigError(f"architecture {self.name!r} does not take the engine option {key!r} "
                                  f"(it takes: {', '.join(sorted(self.options)) or 'none'})")
        return self.model_spec(cfg, **asked)


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    """Add (or replace) an architecture.  Refuses what cannot work: a name that is no string,
    functions that cannot be called, options that the engine does not know."""
    if not isinstance(arch.name, str) or not arch.name:
        raise ConfigError("an architecture needs a name (the string in config.json's `architectures`)")
    if not callable(arch.parse_config) or not callable(arch.model_spec):
        raise ConfigError(f"architecture {arch.name!r}: parse_config and model_spec must be callable")
    unknown = set(arch.options) - KNOWN_OPTIONS
    if unknown:
        raise ConfigError(f"architecture {arch.name!r} lists engine options that do not exist: "
                          f"{', '.join(sorted(unknown))} (known: {', '.join(sorted(KNOWN_OPTIONS))})")
    _ARCHITECTURES[arch.name] = arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def supported_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def architecture_of(raw_config: Mapping[str, Any]) -> Architecture:
    """The architecture named by ``architectures[0]`` of a config.json dictionary."""
    _load_builtin()
    names = raw_config.get("architectures") or []
    name = names[0] if names else "<missing>"
    if name not in _ARCHITECTURES:
        supported = ", ".join(sorted(_ARCHITECTURES))
        raise ConfigError(f"Unsupported architecture {name!r}; supported: {supported}")
    return _ARCHITECTURES[name]


def _load_builtin() -> None:
    if "Qwen3ForCausalLM" not in _ARCHITECTURES:
        from ..models import qwen3
        register_architecture(Architecture(qwen3.ARCHITECTURE, qwen3.parse_config, qwen3.model_spec,
                                           options=frozenset({"window"})))
