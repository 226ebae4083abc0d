"""Model structure as data.

A model is described by a :class:`ModelSpec`: which parts each layer is made of,
with which constants, and in which order the layers run.  Nothing in this file
knows about a concrete architecture; an architecture's builder (for instance
``cretif_b200.config.llama.build_llama_spec``) turns its typed configuration
into a ``ModelSpec`` and the engine assembles the model from it.

The reference engine hard-codes one layer loop (src/model.cu:887-1022) and two
sub-configurations, ``AttentionConfig`` (include/cuinfer/attention.h:20-35) and
``FFNConfig`` (include/cuinfer/ffn.h:25-30).  Here the same separation of
constants from weights is kept, but the loop itself is data.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: a registered ``kind`` and its constants."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):  # params is a dict; hash on a stable rendering
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class BranchSpec:
    """One residual branch of a block: ``h += post_norm(part(norm(h)))``.

    ``role`` is the part's category (``"mixer"`` or ``"feed_forward"``); ``norm`` stands
    before the part and ``post_norm`` after it, and either may be absent.
    """

    role: str
    part: PartSpec
    norm: Optional[PartSpec] = None
    post_norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class LayerSpec:
    """A block: an ordered list of residual branches and the arrangement that wires them.

    The reference's block is two branches, attention then feed-forward, each behind a
    norm of its own (src/model.cu:887-1018); :func:`prenorm_layer` builds exactly that.
    A block may as well have one branch, three, or norms after its parts.
    ``arrangement`` names the registered function that runs the branches
    (``"residual"``: one after the other).  ``prefix`` is the weight-name prefix of the
    layer (``model.layers.3.``).
    """

    prefix: str
    branches: Tuple[BranchSpec, ...]
    arrangement: str = "residual"

    def of_role(self, role: str) -> List[BranchSpec]:
        return [b for b in self.branches if b.role == role]


def prenorm_layer(prefix: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                  feed_forward_norm: PartSpec) -> LayerSpec:
    """``h += mixer(norm1(h))`` then ``h += feed_forward(norm2(h))``."""
    return LayerSpec(prefix, (BranchSpec("mixer", mixer, norm=mixer_norm),
                              BranchSpec("feed_forward", feed_forward, norm=feed_forward_norm)))


@dataclass(frozen=True)
class ScheduleEntry:
    """One visit of a layer when the model runs.

    ``layer`` indexes ``ModelSpec.layers``; the same layer may be visited twice
    (its weights are shared).  ``cache`` names the cache the visit's mixer uses:
    ``None`` gives the visit a cache of its own; an integer ``j`` lets it read
    the cache that schedule entry ``j`` (an earlier one) writes, without writing.
    """

    layer: int
    cache: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    stop_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ValueError("vocab_size and hidden_size must be positive")
        if not self.schedule:
            raise ValueError("the schedule names no layer")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, "
                                 f"but the model has {len(self.layers)} layers")
            for b in self.layers[e.layer].branches:
                if b.role not in ("mixer", "feed_forward"):
                    raise ValueError(f"layer {e.layer}: a branch's role is 'mixer' or "
                                     f"'feed_forward', got {b.role!r}")
            if e.cache is not None:
                if not 0 <= e.cache < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache}, "
                                     "which must be an earlier entry")
                if self.schedule[e.cache].cache is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache}, "
                                     "which itself borrows a cache")
                mine = [b.part for b in self.layers[e.layer].of_role("mixer")]
                theirs = [b.part for b in self.layers[self.schedule[e.cache].layer].of_role("mixer")]
                if len(mine) != len(theirs):
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache}, "
                                     "whose layer has another number of mixers")
