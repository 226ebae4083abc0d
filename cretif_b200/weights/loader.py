"""Weights by tensor name: checked loading, and a seeded random-weights mode.

The reference loads each tensor by name and fails one tensor at a time
(``tensor '<name>' not found``, src/model.cu:76-79; wrong rank :81-85; a shape
mismatch surfaces only later in ``Embedding::forward``, src/embedding.cu:245-251).
Here the model's parts declare every tensor they need (name, shape) up front
and a checkpoint is compared with that manifest in one pass, so a bad file gives
ONE error that lists missing tensors, unexpected tensors and wrong shapes.

Stored dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit
stays 32-bit, integer tables become int32 (float16 and float64 have no kernels
here and are converted to bfloat16 and float32).  Which precision a part
computes in is the part's business, not the loader's.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, Optional, Tuple

import torch

from .safetensors_io import CheckpointError, checkpoint_files, read_tensors, write_tensors


@dataclass(frozen=True)
class WeightSpec:
    """What a part expects of one tensor.

    ``init`` is ``(mean, std)`` of the normal distribution used by the
    random-weights mode; ``integer`` marks index tables.
    """

    shape: Tuple[int, ...]
    init: Tuple[float, float] = (0.0, 0.02)
    integer: bool = False


def _normalise_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise CheckpointError(f"unsupported tensor dtype {t.dtype}")


def load_weights(model_dir: str, manifest: Dict[str, WeightSpec],
                 ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Read every tensor of ``manifest`` from ``model_dir`` (CPU tensors).

    ``ignorable`` names may be present in the file without being used (a stored
    output matrix of a model whose head is tied to the embedding, for instance).
    """
    files = checkpoint_files(model_dir)
    ignorable = set(ignorable)
    missing = sorted(n for n in manifest if n not in files)
    unexpected = sorted(n for n in files if n not in manifest and n not in ignorable)
    by_file: Dict[str, list] = {}
    for name in manifest:
        if name in files:
            by_file.setdefault(files[name], []).append(name)
    tensors: Dict[str, torch.Tensor] = {}
    wrong = []
    for path, names in by_file.items():
        for name, t in read_tensors(path, names).items():
            spec = manifest[name]
            if tuple(t.shape) != tuple(spec.shape):
                wrong.append(f"{name}: expected {list(spec.shape)}, file has {list(t.shape)}")
                continue
            if spec.integer == t.dtype.is_floating_point:
                wrong.append(f"{name}: expected {'an integer' if spec.integer else 'a floating'} "
                             f"tensor, file has {t.dtype}")
                continue
            tensors[name] = _normalise_dtype(t)
    if missing or unexpected or wrong:
        lines = [f"checkpoint in {model_dir!r} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes or types ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise CheckpointError("\n".join(lines))
    return tensors


def _fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def random_weights(manifest: Dict[str, WeightSpec], seed: int,
                   dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Draw every tensor of ``manifest`` from its normal distribution.

    Each tensor has a generator of its own, seeded from ``seed`` and the
    tensor's name, so a tensor's values do not depend on which other tensors
    the model has.  Values are drawn in float32 and then rounded to ``dtype``.
    """
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("random weights are written as bfloat16 or float32")
    out = {}
    for name, spec in manifest.items():
        gen = torch.Generator(device="cpu")
        gen.manual_seed((_fnv1a64(name) ^ (seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF)
        if spec.integer:
            out[name] = torch.randint(0, 2 ** 15, spec.shape, generator=gen, dtype=torch.int32)
            continue
        mean, std = spec.init
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std + mean
        out[name] = t.to(dtype)
    return out


def write_model_folder(model_dir: str, config_json: dict,
                       tensors: Dict[str, torch.Tensor],
                       metadata: Optional[Dict[str, str]] = None) -> None:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir``."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_json, f, indent=2)
        f.write("\n")
    write_tensors(os.path.join(model_dir, "model.safetensors"), tensors,
                  metadata={"format": "pt", **(metadata or {})})
