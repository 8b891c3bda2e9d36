"""The one registry from an architecture's name to its model.

The reference dispatches on config.json's `model_type` through an enum and two `match`
statements (core/src/model_executor/models/model_factory.rs:44-50, :268-333, :155-266).
Here an architecture is registered once with two callables: one that parses config.json
into a typed configuration, one that turns that configuration into a `ModelSpec`
(data that names every part, layer by layer).  Lookup is by `architectures[0]`, then by
`model_type`, both case-insensitive.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List

from .model_config import ConfigError, read_config_json


@dataclass
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]
    build_spec: Callable[[Any], Any]
    aliases: List[str]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec, aliases=()) -> Architecture:
    arch = Architecture(name, parse_config, build_spec, list(aliases))
    for key in [name, *aliases]:
        _ARCHITECTURES[key.lower()] = arch
    return arch


def _load_builtin() -> None:
    from .. import models  # noqa: F401  (importing the package registers the built-in architectures)


def registered_architectures() -> List[str]:
    _load_builtin()
    return sorted({a.name for a in _ARCHITECTURES.values()})


def resolve_architecture(config_dict: Dict[str, Any]) -> Architecture:
    _load_builtin()
    names = list(config_dict.get("architectures") or [])
    if config_dict.get("model_type"):
        names.append(config_dict["model_type"])
    if not names:
        raise ConfigError("config.json names neither 'architectures' nor 'model_type'")
    for n in names:
        arch = _ARCHITECTURES.get(str(n).lower())
        if arch is not None:
            return arch
    raise ConfigError(f"no model is registered for {names}; registered: {', '.join(registered_architectures())}")


def load_model_config(model_dir: str):
    """config.json of a model folder -> (architecture, typed configuration)."""
    d = read_config_json(model_dir)
    arch = resolve_architecture(d)
    return arch, arch.parse_config(d)
