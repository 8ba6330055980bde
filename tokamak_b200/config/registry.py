"""The one registry from an architecture's name to its model.

An architecture is two functions: ``parse_config`` turns the raw ``config.json``
dictionary into a typed configuration, and ``model_spec`` turns that into the
parts, blocks and schedule of the model.  Adding an architecture is adding an
entry (src/tokamak/config.py:20-26 is the reference's whitelist).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[..., Any]
    model_spec: Callable[[Any], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


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
        register_architecture(Architecture(qwen3.ARCHITECTURE, qwen3.parse_config, qwen3.model_spec))
