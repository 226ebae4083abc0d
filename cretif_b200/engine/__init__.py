"""The engine: model assembly, the step function, generation."""
from .engine import Engine, StepError, parse_dtype
from .model import Model, manifest

__all__ = ["Engine", "StepError", "parse_dtype", "Model", "manifest"]
