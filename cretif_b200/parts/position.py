"""Position encodings, applied by a mixer to its queries and keys before the cache write.

``rotary``: each pair of a head's first ``rotary_dim`` channels is rotated by the
angle ``position / theta^(2j / rotary_dim)`` (src/kernels/elementwise.cu:232-258).
``pairing`` says which channels form pair ``j``: ``"interleaved"`` is the
reference's ``(2j, 2j+1)``; ``"half"`` is ``(j, j + rotary_dim/2)``, the layout of
query/key rows in config.json + safetensors checkpoints (the reference's weight
files carry those rows permuted so that its interleaved rotation gives the same
function).  Angles, cosines and sines are computed once on the host in 64-bit and
kept as a 32-bit table ``[positions, rotary_dim/2]`` that every kernel reads, so a
position's rotation is the same in every step shape.

``none``: queries and keys stay as they are.

Interface of a position part: ``prepare(max_positions)`` builds what depends on the longest
sequence; ``encode(qkv, ctx, nh, nkv, hd)`` position-encodes the queries and keys of the
packed ``[T, (nh + 2·nkv)·hd]`` buffer in place.  Storing keys and values in the cache is the
mixer's job, not the encoding's.  A part whose encoding is a rotation by a table may also
offer ``rotary_table() -> (cos, sin, pairing, rotary_dim)``; a mixer can then hand the table
to kernels that rotate inside a product's epilogue or together with the cache write.  A part
that offers it promises that ``encode`` is exactly that rotation.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..csrc import ops
from .base import Part, register_part

_TABLES: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


def rotary_table(theta: float, rot_dim: int, positions: int, device):
    key = (float(theta), rot_dim, positions, str(device))
    if key not in _TABLES:
        j = torch.arange(rot_dim // 2, dtype=torch.float64)
        freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * j / rot_dim)
        ang = torch.arange(positions, dtype=torch.float64)[:, None] * freq[None, :]
        _TABLES[key] = (torch.cos(ang).to(torch.float32).to(device).contiguous(),
                        torch.sin(ang).to(torch.float32).to(device).contiguous())
    return _TABLES[key]


@register_part("position", "rotary")
class Rotary(Part):
    """params: ``theta``, ``rotary_dim``, ``pairing`` ("half" or "interleaved")."""

    graph_safe = True

    def load(self, tensors):
        self.theta = float(self.params["theta"])
        self.rot_dim = int(self.params["rotary_dim"])
        pairing = self.params.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing must be 'half' or 'interleaved', got {pairing!r}")
        if self.rot_dim % 2:
            raise ValueError("rotary_dim must be even")
        self.pairing = 1 if pairing == "interleaved" else 0
        self._table = None

    def prepare(self, max_positions: int) -> None:
        self._table = rotary_table(self.theta, self.rot_dim, max_positions, self.device)

    def rotary_table(self):
        cos, sin = self._table
        return cos, sin, self.pairing, self.rot_dim

    def encode(self, qkv, ctx, nh, nkv, hd):
        cos, sin = self._table
        ops.rope_kv_append(qkv, cos, sin, self.pairing, self.rot_dim, nh, nkv, hd, ctx.tok_pos,
                           write_cache=False, fault=ctx.fault, rotate_k_in_place=True)


@register_part("position", "none")
class NoPosition(Part):
    """Leaves queries and keys as they are."""

    graph_safe = True

    def prepare(self, max_positions: int) -> None:
        pass

    def encode(self, qkv, ctx, nh, nkv, hd):
        pass
