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

from ..config.spec import BranchSpec, ModelSpec, PartSpec
from ..parts.base import LayerCache, Part, StepContext, build_part, lookup_part
from ..weights.loader import WeightSpec


@dataclass
class Branch:
    """One built residual branch of a layer: ``h += post_norm(part(norm(h)))``."""

    role: str                      # "mixer" or "feed_forward"
    part: Part
    norm: Optional[Part] = None
    post_norm: Optional[Part] = None

    def parts(self) -> List[Part]:
        return [p for p in (self.norm, self.part, self.post_norm) if p is not None]


@dataclass
class Layer:
    prefix: str
    branches: List[Branch]
    run: Callable


def _with(spec: PartSpec, **extra) -> PartSpec:
    return PartSpec(spec.kind, {**spec.params, **extra})


def _branch_specs(bs: BranchSpec):
    """(category, PartSpec) of a branch's parts, in the order they are built and loaded."""
    if bs.norm is not None:
        yield "norm", bs.norm
    yield bs.role, bs.part
    if bs.post_norm is not None:
        yield "norm", bs.post_norm


def _part_specs(spec: ModelSpec):
    """Every (category, PartSpec, name prefix) of the model, in a fixed order."""
    yield "embedding", _with(spec.embedding, vocab_size=spec.vocab_size), ""
    for layer in spec.layers:
        for bs in layer.branches:
            for category, pspec in _branch_specs(bs):
                yield category, pspec, layer.prefix
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
        # every part is built in the order of _part_specs, which is also the order of loading
        built = [build_part(category, pspec, H, dtype, device)
                 for category, pspec, _ in _part_specs(spec)]
        self._parts: List[Part] = built
        it = iter(built)
        self.embedding = next(it)
        self.layers: List[Layer] = []
        for ls in spec.layers:
            branches = []
            for bs in ls.branches:
                norm = next(it) if bs.norm is not None else None
                part = next(it)
                post = next(it) if bs.post_norm is not None else None
                branches.append(Branch(bs.role, part, norm, post))
            self.layers.append(Layer(ls.prefix, branches,
                                     lookup_part("arrangement", ls.arrangement)))
        self.final_norm = next(it)
        self.head = next(it)

    def parts(self) -> List[Part]:
        """Every part of the model: embedding, each layer's branches in order, final norm, head."""
        return list(self._parts)

    @property
    def graph_safe(self) -> bool:
        """Whether every part allows its steps to be captured as CUDA graphs."""
        return all(getattr(p, "graph_safe", False) for p in self._parts)

    # -- weights ---------------------------------------------------------------
    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand each part its tensors (CPU, by full name) and let it place them."""
        for part, (category, pspec, prefix) in zip(self._parts, _part_specs(self.spec)):
            specs = lookup_part(category, pspec.kind).weight_specs(pspec.params,
                                                                   self.spec.hidden_size)
            part.load({key: tensors[prefix + name] for key, (name, _) in specs.items()})
        if self.spec.head.params.get("tied"):
            self.head.tie(self.embedding)

    def prepare(self, max_positions: int) -> None:
        """Let every part build what depends on the longest sequence (position tables)."""
        for part in self._parts:
            if hasattr(part, "prepare"):
                part.prepare(max_positions)

    # -- cache -------------------------------------------------------------------
    def cache_requests(self) -> Dict[Tuple[int, int], Any]:
        """cache id → what its part keeps between steps.  A cache id is (index of the owning
        schedule entry, index of the branch in its layer); only entries that own their cache
        (``ScheduleEntry.cache is None``) appear."""
        out = {}
        for i, entry in enumerate(self.spec.schedule):
            if entry.cache is None:
                for k, br in enumerate(self.layers[entry.layer].branches):
                    if hasattr(br.part, "cache_request"):
                        out[(i, k)] = br.part.cache_request()
        return out

    def layer_caches(self, i: int, cache) -> List[Optional[LayerCache]]:
        """What each branch of schedule entry ``i`` is handed: its own cache, the cache of the
        entry it borrows from (read-only), or None for a part that keeps nothing."""
        entry = self.spec.schedule[i]
        owner = i if entry.cache is None else entry.cache
        views: List[Optional[LayerCache]] = []
        for k, br in enumerate(self.layers[entry.layer].branches):
            cid = (owner, k)
            if entry.cache is not None and br.role == "mixer":
                # the k-th mixer of this layer reads the k-th mixer's cache of the owner's layer
                mine = [j for j, b in enumerate(self.layers[entry.layer].branches)
                        if b.role == "mixer"]
                theirs = [j for j, b in enumerate(
                    self.layers[self.spec.schedule[owner].layer].branches) if b.role == "mixer"]
                cid = (owner, theirs[mine.index(k)])
            kv = cache.kv_view(cid) if cache.has_kv(cid) else None
            state = cache.state_view(cid) if cache.has_state(cid) else None
            views.append(None if kv is None and state is None
                         else LayerCache(kv=kv, state=state, writes=entry.cache is None))
        return views

    # -- one step ------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """Run the scheduled layers on the step's tokens; logits [rows, vocab] float32
        at ``want_rows`` (token indices), or at every token when it is None."""
        h = self.embedding.forward(ctx.tok_ids, ctx)
        pending = None
        for i, entry in enumerate(self.spec.schedule):
            layer = self.layers[entry.layer]
            pending = layer.run(layer, h, pending, ctx, self.layer_caches(i, cache))
        if want_rows is not None and want_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        if hasattr(self.head, "forward_from_residual"):
            logits = self.head.forward_from_residual(h, pending, self.final_norm, want_rows, ctx)
            if logits is not None:
                return logits
        n = self.final_norm.forward(h, pending, rows=want_rows, write_h=False)
        return self.head.forward(n, ctx)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self._parts)
