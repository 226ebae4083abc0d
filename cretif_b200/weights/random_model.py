"""The random-weights mode: a model folder from a configuration and a seed.

Matrices are drawn from N(0, 0.02) and norm weights from 1 + N(0, 0.02); each part
declares the distribution of its tensors in its ``weight_specs``.  The folder holds
``config.json`` and ``model.safetensors`` and is read back like any checkpoint.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.registry import architecture_name, resolve_architecture
from .loader import random_weights, write_model_folder


def write_random_model(model_dir: str, config_json: Dict[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Write a model folder for ``config_json`` (a config.json as a dict) with seeded
    random weights stored as ``dtype`` (bfloat16 or float32)."""
    from ..engine.model import manifest   # parts are registered on import
    arch = resolve_architecture(architecture_name(config_json))
    cfg = arch.config_from_dict(config_json)
    spec = arch.build_spec(cfg)
    spec.validate()
    names, _ = manifest(spec)
    tensors = random_weights(names, seed, dtype)
    out_cfg = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(config_json)
    out_cfg.setdefault("torch_dtype", "bfloat16" if dtype == torch.bfloat16 else "float32")
    write_model_folder(model_dir, out_cfg, tensors, metadata={"seed": str(seed)})
