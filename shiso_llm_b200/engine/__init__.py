"""The step function, the scheduler above it and the user-facing entry point."""

from .batch import StepBuilder, StepEntry, StepMeta
from .core import Engine, EngineOptions, parse_dtype

__all__ = ["Engine", "EngineOptions", "StepBuilder", "StepEntry", "StepMeta", "parse_dtype"]
