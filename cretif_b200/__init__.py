"""cretif_b200 — a small, whole Llama inference library for NVIDIA B200 (sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens on one
GPU: typed configuration and architecture registry, checked weight loading, parts
(norm, position encoding, attention, feed-forward) assembled layer by layer from the
configuration, a block-pooled cache with one slot per sequence, one step function,
a generation loop with sampling, and a trace-replay program — on hand-written CUDA
kernels, in bfloat16 and in true 32-bit.
"""
from . import config, weights, cache  # noqa: F401

__version__ = "0.1.0"


def load(model_dir, dtype="bfloat16", max_tokens=8192, device="cuda:0", **kw):
    """Load a model folder onto a GPU; returns an :class:`~cretif_b200.engine.Engine`."""
    from .engine import Engine
    return Engine(model_dir, dtype=dtype, max_tokens=max_tokens, device=device, **kw)
