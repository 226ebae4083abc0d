"""Typed configurations, the architecture registry and the model structure data."""
from .registry import (ConfigError, architecture_name, load_config, read_config_json,
                       register_architecture, registered_architectures, resolve_architecture)
from .spec import BranchSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, prenorm_layer
from .llama import LlamaConfig, build_llama_spec, llama_config_from_dict
from .presets import PRESETS, preset

__all__ = [
    "ConfigError", "architecture_name", "load_config", "read_config_json",
    "register_architecture", "registered_architectures", "resolve_architecture",
    "BranchSpec", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "prenorm_layer",
    "LlamaConfig", "build_llama_spec", "llama_config_from_dict", "PRESETS", "preset",
]
