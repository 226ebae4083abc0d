"""One registry from an architecture's name to its configuration class and builder.

The reference stores the architecture string only as a metadata key prefix
(src/gguf_parser.cpp:694-740) and runs the same code for every file; here the
name in ``config.json`` (``architectures[0]``) picks the typed configuration and
the function that turns it into a :class:`~cretif_b200.config.spec.ModelSpec`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .spec import ModelSpec


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, build_spec) -> None:
    """Register ``name`` (as it appears in ``architectures``) with its two functions."""
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {registered_architectures()}") from None


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def architecture_name(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if isinstance(archs, str):
        return archs
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json has no 'architectures' list naming the model class")
    return archs[0]


def load_config(model_dir: str):
    """Read ``model_dir/config.json`` → ``(architecture, typed config, ModelSpec)``."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(architecture_name(raw))
    cfg = arch.config_from_dict(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    return arch, cfg, spec
