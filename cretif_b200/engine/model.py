"""Assembling a model from a ModelSpec, and running its layers for one step.

The model is a list of layers built from registered parts, run in the order the
spec's schedule gives.  ``manifest`` collects every tensor the parts declare, which
is what a checkpoint is checked against and what the random-weights mode draws.
The forward pass is the reference's (src/model.cu:859-1039): embedding, then per
scheduled layer its arrangement, then the final norm and the head — but only on the
rows whose logits are wanted.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Set, Tuple

import torch

from ..config.spec import ModelSpec, PartSpec
from ..parts.base import LayerCache, Part, StepContext, build_part, lookup_part
from ..weights.loader import WeightSpec


@dataclass
class Layer:
    prefix: str
    mixer_norm: Part
    mixer: Part
    feed_forward_norm: Part
    feed_forward: Part
    run: Callable


def _with(spec: PartSpec, **extra) -> PartSpec:
    return PartSpec(spec.kind, {**spec.params, **extra})


def _part_specs(spec: ModelSpec):
    """Every (category, PartSpec, name prefix) of the model, in a fixed order."""
    yield "embedding", _with(spec.embedding, vocab_size=spec.vocab_size), ""
    for layer in spec.layers:
        yield "norm", layer.mixer_norm, layer.prefix
        yield "mixer", layer.mixer, layer.prefix
        yield "norm", layer.feed_forward_norm, layer.prefix
        yield "feed_forward", layer.feed_forward, layer.prefix
    yield "norm", spec.final_norm, ""
    yield "head", _with(spec.head, vocab_size=spec.vocab_size), ""


def manifest(spec: ModelSpec) -> Tuple[Dict[str, WeightSpec], Set[str]]:
    """All tensors of the model by full name, and names a file may hold unused."""
    out: Dict[str, WeightSpec] = {}
    for category, pspec, prefix in _part_specs(spec):
        cls = lookup_part(category, pspec.kind)
        for _, (name, wspec) in cls.weight_specs(pspec.params, spec.hidden_size).items():
            full = prefix + name
            if full in out and out[full] != wspec:
                raise ValueError(f"tensor {full!r} is declared twice with different shapes")
            out[full] = wspec
    ignorable: Set[str] = set()
    if spec.head.params.get("tied") and spec.head.params.get("name"):
        ignorable.add(spec.head.params["name"])
    return out, ignorable


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the compute dtype must be float32 or bfloat16, got {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        H = spec.hidden_size
        self.embedding = build_part("embedding", _with(spec.embedding, vocab_size=spec.vocab_size),
                                    H, dtype, device)
        self.layers: List[Layer] = []
        for ls in spec.layers:
            self.layers.append(Layer(
                prefix=ls.prefix,
                mixer_norm=build_part("norm", ls.mixer_norm, H, dtype, device),
                mixer=build_part("mixer", ls.mixer, H, dtype, device),
                feed_forward_norm=build_part("norm", ls.feed_forward_norm, H, dtype, device),
                feed_forward=build_part("feed_forward", ls.feed_forward, H, dtype, device),
                run=lookup_part("arrangement", ls.arrangement)))
        self.final_norm = build_part("norm", spec.final_norm, H, dtype, device)
        self.head = build_part("head", _with(spec.head, vocab_size=spec.vocab_size), H, dtype,
                               device)

    @property
    def graph_safe(self) -> bool:
        """Whether every part allows its steps to be captured as CUDA graphs."""
        parts = [self.embedding, self.final_norm, self.head]
        for layer in self.layers:
            parts += [layer.mixer_norm, layer.mixer, layer.feed_forward_norm, layer.feed_forward]
        return all(getattr(p, "graph_safe", False) for p in parts)

    # -- weights ---------------------------------------------------------------
    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand each part its tensors (CPU, by full name) and let it place them."""
        def give(part: Part, category: str, pspec: PartSpec, prefix: str):
            specs = lookup_part(category, pspec.kind).weight_specs(pspec.params,
                                                                   self.spec.hidden_size)
            part.load({key: tensors[prefix + name] for key, (name, _) in specs.items()})
        s = self.spec
        give(self.embedding, "embedding", _with(s.embedding, vocab_size=s.vocab_size), "")
        for layer, ls in zip(self.layers, s.layers):
            give(layer.mixer_norm, "norm", ls.mixer_norm, ls.prefix)
            give(layer.mixer, "mixer", ls.mixer, ls.prefix)
            give(layer.feed_forward_norm, "norm", ls.feed_forward_norm, ls.prefix)
            give(layer.feed_forward, "feed_forward", ls.feed_forward, ls.prefix)
        give(self.final_norm, "norm", s.final_norm, "")
        give(self.head, "head", _with(s.head, vocab_size=s.vocab_size), "")
        if s.head.params.get("tied"):
            self.head.tie(self.embedding)

    def prepare(self, max_positions: int) -> None:
        """Build what depends on the longest sequence (position tables)."""
        for layer in self.layers:
            if hasattr(layer.mixer, "prepare"):
                layer.mixer.prepare(max_positions)

    # -- cache -------------------------------------------------------------------
    def cache_requests(self) -> Dict[int, Any]:
        """cache id (index of the owning schedule entry) → what its mixer keeps."""
        out = {}
        for i, entry in enumerate(self.spec.schedule):
            if entry.cache is None:
                mixer = self.layers[entry.layer].mixer
                out[i] = mixer.cache_request() if hasattr(mixer, "cache_request") else None
        return out

    # -- one step ------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """Run the scheduled layers on the step's tokens; logits [rows, vocab] float32
        at ``want_rows`` (token indices), or at every token when it is None."""
        sk = getattr(self, "step_kernel", None)
        if sk is not None and sk.takes(ctx):
            return sk.run(ctx, want_rows)            # the whole step in one launch
        h = self.embedding.forward(ctx.tok_ids, ctx)
        pending = None
        for i, entry in enumerate(self.spec.schedule):
            cid = i if entry.cache is None else entry.cache
            view = LayerCache(kv=cache.kv_view(cid) if cache.has_kv(cid) else None,
                              state=cache.state_view(cid) if cache.has_state(cid) else None,
                              writes=entry.cache is None)
            layer = self.layers[entry.layer]
            pending = layer.run(layer, h, pending, ctx, view)
        if want_rows is not None and want_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        if hasattr(self.head, "forward_from_residual"):
            logits = self.head.forward_from_residual(h, pending, self.final_norm, want_rows, ctx)
            if logits is not None:
                return logits
        n = self.final_norm.forward(h, pending, rows=want_rows, write_h=False)
        return self.head.forward(n, ctx)

    def weight_bytes(self) -> int:
        total = self.embedding.weight_bytes() + self.final_norm.weight_bytes() \
            + self.head.weight_bytes()
        for layer in self.layers:
            total += (layer.mixer_norm.weight_bytes() + layer.mixer.weight_bytes()
                      + layer.feed_forward_norm.weight_bytes() + layer.feed_forward.weight_bytes())
        return total
