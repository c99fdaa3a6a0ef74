"""One registry from an architecture's name to its configuration and plan.

``config.json`` names the model class in ``architectures[0]``; that string is
the key.  An entry holds the typed configuration class (which reads the
architecture's own config.json keys) and a function that turns a configuration
into a ``ModelPlan``.  The reference resolves a family with a chain of
``Family::describes(config)`` arms that ends in ``UnknownArchitecture``
(crates/shiso-runtime/src/model_factory.rs:784-813); here the chain is a table.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping

from ..parts.plan import ModelPlan
from .errors import ConfigError, ConfigMissing, InvalidValue, UnknownArchitecture


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_plan: Callable[[Any], ModelPlan]
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_plan, model_types=()) -> Architecture:
    """Adds an architecture.  ``config_class`` needs ``from_dict`` and ``to_dict``."""
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is registered already")
    arch = Architecture(name, config_class, build_plan, tuple(model_types))
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(document: Mapping[str, Any]) -> Architecture:
    """Picks the registry entry a config.json document names."""
    names = document.get("architectures")
    if names is not None:
        if not isinstance(names, list) or not names or not isinstance(names[0], str):
            raise InvalidValue("architectures", names, "expected a non-empty list of names")
        arch = _ARCHITECTURES.get(names[0])
        if arch is None:
            raise UnknownArchitecture(names[0], registered_architectures())
        return arch
    model_type = document.get("model_type")
    if model_type is None:
        raise ConfigMissing("architectures")
    for arch in _ARCHITECTURES.values():
        if model_type in arch.model_types:
            return arch
    raise UnknownArchitecture(str(model_type), registered_architectures())


def read_config_document(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            document = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(document, dict):
        raise ConfigError(f"{path}: expected a JSON object at the top level")
    return document


def load_config(model_dir: str):
    """Reads ``config.json`` of a model folder: (architecture entry, typed config)."""
    document = read_config_document(model_dir)
    arch = architecture_of(document)
    return arch, arch.config_class.from_dict(document)


def plan_from_document(document: Mapping[str, Any]) -> tuple[Architecture, Any, ModelPlan]:
    arch = architecture_of(document)
    config = arch.config_class.from_dict(document)
    return arch, config, arch.build_plan(config)
