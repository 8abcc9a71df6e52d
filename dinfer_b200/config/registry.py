"""One registry from an architecture's name (``config.json``'s ``architectures[0]``) to the
pair that makes a model of it: the typed configuration and the function that turns that
configuration into a ``ModelSpec`` (the list of layers and parts).

The reference picks its model at compile time by a cargo feature
(bins/dinfer/Cargo.toml:13-20, bins/dinfer/src/main.rs:6-18) and never reads
``architectures``; here the name in the file decides.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    # config.json dictionary -> typed configuration (raises ConfigError)
    parse_config: Callable[[Dict[str, Any]], Any]
    # typed configuration -> parts.spec.ModelSpec
    build_spec: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_dict: Dict[str, Any]) -> Architecture:
    """The registered architecture that ``config.json`` names."""
    _ensure_builtin()
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"config.json: architecture {name!r} is not registered "
            f"(registered: {', '.join(registered_architectures())})")
    return _ARCHITECTURES[name]


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from ..models import qwen3  # noqa: F401  (registers itself)
