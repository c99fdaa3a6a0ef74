"""Typed configurations and the architecture registry."""

from .errors import ConfigError, ConfigMissing, InvalidValue, UnknownArchitecture, UnsupportedShape
from .registry import (
    Architecture,
    architecture_of,
    load_config,
    plan_from_document,
    read_config_document,
    register_architecture,
    registered_architectures,
    unregister_architecture,
)
from . import lfm2  # registers Lfm2ForCausalLM
from .lfm2 import Lfm2Config, feed_forward_width

__all__ = [
    "Architecture",
    "ConfigError",
    "ConfigMissing",
    "InvalidValue",
    "Lfm2Config",
    "UnknownArchitecture",
    "UnsupportedShape",
    "architecture_of",
    "feed_forward_width",
    "load_config",
    "plan_from_document",
    "read_config_document",
    "register_architecture",
    "registered_architectures",
    "unregister_architecture",
]
