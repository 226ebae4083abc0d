"""Parts a model is put together from: embedding, norms, mixers, feed-forwards,
position encodings, heads, and the arrangements that wire them into a block."""
from .base import (LayerCache, Part, StepContext, build_part, lookup_part, register_part,
                   registered_parts)
from . import attention, block, embedding, mlp, norm, position  # noqa: F401  (register the parts)

__all__ = ["LayerCache", "Part", "StepContext", "build_part", "lookup_part", "register_part",
           "registered_parts"]
