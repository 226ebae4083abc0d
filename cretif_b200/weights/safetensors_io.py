"""Reading and writing the safetensors container (8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}``, then raw data).

This replaces the reference's GGUF parser (src/gguf_parser.cpp:524-618, tensor
lookup by name at :773-782) for the one job the engine needs: tensors by name.
Like the parser, it refuses data that reaches beyond the end of the file
(src/gguf_parser.cpp:786-792).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch


class CheckpointError(ValueError):
    """A weight file that cannot be read, or that does not fit the model."""


_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def read_header(path: str) -> Tuple[Dict[str, dict], int]:
    """Return ``(entries, data_start)`` of a safetensors file after checking its bounds."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise CheckpointError(f"{path}: too short to hold a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise CheckpointError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{path}: header is not valid JSON ({e})") from None
    if not isinstance(header, dict):
        raise CheckpointError(f"{path}: header is not a JSON object")
    header.pop("__metadata__", None)
    data_start = 8 + n
    for name, ent in header.items():
        try:
            dt, shape, (b, e) = ent["dtype"], ent["shape"], ent["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise CheckpointError(f"{path}: malformed entry for tensor {name!r}") from None
        if dt not in _DTYPES:
            raise CheckpointError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
        want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dt][1] if shape else _DTYPES[dt][1]
        if b < 0 or e < b or e - b != want:
            raise CheckpointError(f"{path}: tensor {name!r} of shape {shape} and dtype {dt} "
                                  f"needs {want} bytes but its offsets span {e - b}")
        if data_start + e > size:
            raise CheckpointError(f"{path}: tensor {name!r} reaches beyond the end of the file")
    return header, data_start


def read_tensors(path: str, names: Optional[Iterable[str]] = None) -> Dict[str, torch.Tensor]:
    """Read tensors (all, or the ones in ``names``) with the dtype they are stored in."""
    header, start = read_header(path)
    wanted = set(header) if names is None else set(names)
    buf = np.memmap(path, dtype=np.uint8, mode="r")
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(wanted):
        ent = header[name]
        dtype, _ = _DTYPES[ent["dtype"]]
        b, e = ent["data_offsets"]
        raw = torch.from_numpy(np.array(buf[start + b:start + e]))  # owned copy
        out[name] = raw.view(dtype).reshape(ent["shape"])
    del buf
    return out


def write_tensors(path: str, tensors: Dict[str, torch.Tensor],
                  metadata: Optional[Dict[str, str]] = None) -> None:
    """Write ``tensors`` (CPU, contiguous after this call) in name order."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise CheckpointError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + raw.nbytes]}
        offset += raw.nbytes
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw.tobytes())
    os.replace(tmp, path)


def checkpoint_files(model_dir: str) -> Dict[str, str]:
    """Map tensor name → file for a model folder (one file, or an index of shards)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        header, _ = read_header(single)
        return {name: single for name in header}
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            try:
                weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise CheckpointError(f"{index}: no 'weight_map' object") from None
        out = {}
        for name, shard in weight_map.items():
            p = os.path.join(model_dir, shard)
            if not os.path.isfile(p):
                raise CheckpointError(f"{index}: shard {shard!r} of tensor {name!r} is missing")
            out[name] = p
        return out
    raise CheckpointError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir!r}")
