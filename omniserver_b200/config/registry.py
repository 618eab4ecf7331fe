"""One registry from an architecture's name (``architectures[0]`` of config.json) to its model.

The reference has no registry: its adapter class is imported directly
(omniserve/models/__init__.py:3-6).  An entry is a pair: how to read the typed
configuration from the config.json dictionary, and how to turn it into a ModelSpec.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Tuple

from .model_config import ConfigError, read_config_dict

_ARCHITECTURES: Dict[str, Tuple[Callable[[dict], Any], Callable[[Any], Any]]] = {}


def register_architecture(name: str, parse_config: Callable[[dict], Any], build_spec: Callable[[Any], Any]) -> None:
    _ARCHITECTURES[name] = (parse_config, build_spec)


def known_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    from .. import models  # noqa: F401  (registers the built-in architecture)


def resolve(config_dict: dict):
    """(typed config, ModelSpec) for a config.json dictionary."""
    _ensure_builtin()
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config: 'architectures' (a non-empty list) is missing")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; this engine knows: {', '.join(sorted(_ARCHITECTURES))}")
    parse, build = _ARCHITECTURES[name]
    cfg = parse(config_dict)
    return cfg, build(cfg)


def resolve_dir(model_dir: str):
    return resolve(read_config_dict(model_dir))
