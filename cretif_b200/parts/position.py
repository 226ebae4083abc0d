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

``none``: keys and values are stored as they are.

Interface: ``rotate_and_store(qkv, ctx, cache, nh, nkv, hd)`` rotates q in place in
the packed ``[T, (nh + 2·nkv)·hd]`` buffer and writes rotated k, and v, into the
block cache of ``cache.kv`` (unless the visit only borrows that cache).
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

    def rotate_and_store(self, qkv, ctx, cache, nh, nkv, hd):
        cos, sin = self._table
        kv = cache.kv
        ops.rope_kv_append(qkv, cos, sin, self.pairing, self.rot_dim, nh, nkv, hd, ctx.tok_pos,
                           ctx.tok_seq, ctx.seq_slot, kv.table, kv.k, kv.v, kv.block_tokens,
                           cache.writes, ctx.fault)


@register_part("position", "none")
class NoPosition(Part):
    """Stores keys and values unrotated."""

    graph_safe = True

    def load(self, tensors):
        self._table = None

    def prepare(self, max_positions: int) -> None:
        z = torch.zeros((1, 1), dtype=torch.float32, device=self.device)
        self._table = (z, z)

    def rotate_and_store(self, qkv, ctx, cache, nh, nkv, hd):
        cos, sin = self._table
        kv = cache.kv
        ops.rope_kv_append(qkv, cos, sin, 0, 0, nh, nkv, hd, ctx.tok_pos, ctx.tok_seq,
                           ctx.seq_slot, kv.table, kv.k, kv.v, kv.block_tokens, cache.writes,
                           ctx.fault)
