"""Interfaces of the parts a model is assembled from, and their registries.

A part is a small class that owns its constants (given as ``params``) and its
weights, and knows nothing about the model it sits in.  There are six kinds:

===============  =============================================================
kind             interface
===============  =============================================================
embedding        ``forward(ids[T] int32, ctx) -> h[T, H] float32``
norm             ``forward(h, delta, rows=None, write_h=True) -> n[R, H]``:
                 ``h += delta`` (when given), ``n = norm(h)`` in the compute dtype
mixer            ``forward(x[T, H], ctx, cache) -> y[T, H]`` (any float dtype);
                 ``cache_request()`` says what it keeps between steps
feed_forward     ``forward(x[T, H], ctx) -> y[T, H]``
position         used by a mixer; ``rotate_and_store(qkv, ctx, kv_view, ...)``
head             ``forward(n[R, H], ctx) -> logits[R, V] float32``
===============  =============================================================

Every part class also has ``weight_specs(params, hidden_size)``: a dict from a
short key to ``(tensor name relative to the part's prefix, WeightSpec)``, which is
how the loader learns the names and shapes a checkpoint must have, and
``load(tensors)`` which receives the CPU tensors under the same short keys.

The residual stream ``h`` is float32 in every mode; ``x`` and ``n`` have the
compute dtype (float32 or bfloat16).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch

from ..config.spec import PartSpec
from ..weights.loader import WeightSpec

_KINDS = ("embedding", "norm", "mixer", "feed_forward", "position", "head", "arrangement")
_REGISTRY: Dict[str, Dict[str, Any]] = {k: {} for k in _KINDS}


def register_part(category: str, kind: str):
    """Class (or function, for arrangements) decorator: ``@register_part("mixer", "attention")``."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; there are {_KINDS}")

    def deco(obj):
        _REGISTRY[category][kind] = obj
        return obj
    return deco


def lookup_part(category: str, kind: str):
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise KeyError(f"no {category} part of kind {kind!r} is registered; "
                       f"registered: {sorted(_REGISTRY.get(category, {}))}") from None


def registered_parts(category: str):
    return sorted(_REGISTRY[category])


@dataclass
class StepContext:
    """What one step looks like, on the device, for every part to read.

    ``T`` tokens of ``B`` sequences are packed one sequence after another.
    All index tensors are int32 on the device.
    """

    T: int
    B: int
    tok_ids: torch.Tensor        # [T] token ids
    tok_pos: torch.Tensor        # [T] absolute position of each token
    tok_seq: torch.Tensor        # [T] index of the token's sequence within the batch
    seq_slot: torch.Tensor       # [B] cache slot of each sequence
    seq_start: torch.Tensor      # [B] tokens cached before this step
    cu_seqlens: torch.Tensor     # [B + 1] offsets of the sequences in the packed tokens
    is_decode: bool              # every sequence brings exactly one token
    max_new: int                 # host copy: most tokens one sequence brings
    max_context: int             # host copy: longest context after this step
    fault: torch.Tensor          # [1] int32 status word the kernels OR their faults into
    dtype: torch.dtype           # compute dtype of the run
    device: torch.device
    seq_slot_host: Tuple[int, ...] = ()
    seq_start_host: Tuple[int, ...] = ()
    seq_new_host: Tuple[int, ...] = ()
    extras: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerCache:
    """The cache a mixer is handed for one visit of its layer."""

    kv: Optional[Any] = None          # cretif_b200.cache.KVView
    state: Optional[torch.Tensor] = None   # [max_slots, *shape]
    writes: bool = True               # False: the visit borrows another visit's cache


class Part:
    """Base of all parts: constants, weights, device placement.

    ``graph_safe`` says that ``forward`` only launches work on the current stream — no
    host reads of device data, no host-side state that changes from step to step — so a step
    through the part can be captured as a CUDA graph.  It is False unless a part says
    otherwise; a model with one part that is not graph-safe simply runs every step eagerly.
    """

    graph_safe = False

    def __init__(self, params: Dict[str, Any], hidden_size: int, dtype: torch.dtype, device):
        self.params = dict(params)
        self.hidden_size = hidden_size
        self.dtype = dtype
        self.device = torch.device(device)

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], hidden_size: int
                     ) -> Dict[str, Tuple[str, WeightSpec]]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    # helpers for subclasses
    def _matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A weight matrix in the compute dtype on the device (bf16 → f32 is exact)."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def _vector32(self, t: torch.Tensor) -> torch.Tensor:
        """A per-channel weight in float32: norms are computed in 32-bit."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return 0


def build_part(category: str, spec: PartSpec, hidden_size: int, dtype, device) -> Part:
    return lookup_part(category, spec.kind)(spec.params, hidden_size, dtype, device)
