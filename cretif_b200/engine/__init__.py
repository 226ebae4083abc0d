"""The engine: model assembly, the step function, generation."""
from .engine import Engine, StepError, parse_dtype
from .generate import GenerationLoop, GenerationResult, generate
from .model import Model, manifest

__all__ = ["Engine", "StepError", "parse_dtype", "GenerationLoop", "GenerationResult",
           "generate", "Model", "manifest"]
