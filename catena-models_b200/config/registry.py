"""The one registry from an architecture's name to its configuration class and its model.

catena-models resolves `general.architecture` through an enum and a match
(src/checkpoint.rs:487-497, src/catena.rs:109-118); here the table is open so that a test or
a later architecture registers itself without touching the engine:

    register_architecture("name", ConfigClass, define)

`ConfigClass.from_dict(dict)` returns the typed configuration; `define(config)` returns the
`ModelDefinition` (engine/definition.py) that the engine builds layer by layer.
"""
from __future__ import annotations

import dataclasses

from .base import ConfigError, architecture_name, read_config_json


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    define: callable


_ARCHITECTURES = {}


def register_architecture(name, config_class, define, replace=False):
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, define)


def architectures():
    return sorted(_ARCHITECTURES)


def resolve(name):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{name}'; registered: {', '.join(architectures()) or 'none'}"
        ) from None


def config_from_dict(data, where="config.json"):
    """(Architecture, typed config) for a dict read from config.json."""
    arch = resolve(architecture_name(data))
    return arch, arch.config_class.from_dict(data, where)


def config_from_folder(folder):
    return config_from_dict(read_config_json(folder), where=f"{folder}/config.json")
