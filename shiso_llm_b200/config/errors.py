"""Typed refusals raised while a model folder's ``config.json`` is read.

The reference refuses bad input loudly instead of substituting a default
(AGENTS.md:141-142) and names the offending key in a typed error
(crates/shiso-core/src/error.rs: UnknownArch, ConfigMissing, InvalidValue,
ShapeMismatch).  The classes here carry the same information.
"""

from __future__ import annotations


class ConfigError(ValueError):
    """Base of every refusal made while reading a configuration."""


class UnknownArchitecture(ConfigError):
    """The document names an architecture no registry entry answers to."""

    def __init__(self, name: str, known: list[str]):
        self.name = name
        self.known = list(known)
        super().__init__(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(known)) or '(none)'}"
        )


class ConfigMissing(ConfigError):
    """A key the architecture needs is absent from config.json."""

    def __init__(self, key: str):
        self.key = key
        super().__init__(f"config.json has no key {key!r}")


class InvalidValue(ConfigError):
    """A key is present but its value cannot describe a model."""

    def __init__(self, key: str, value, why: str):
        self.key = key
        self.value = value
        super().__init__(f"config.json: {key} = {value!r}: {why}")


class UnsupportedShape(ConfigError):
    """A size is legal for the architecture but no kernel here takes it."""

    def __init__(self, what: str, value, why: str):
        self.what = what
        self.value = value
        super().__init__(f"unsupported {what} = {value!r}: {why}")
