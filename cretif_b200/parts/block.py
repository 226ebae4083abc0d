"""Arrangements: how a layer's norms, mixer and feed-forward are wired.

An arrangement is a function ``run(layer, h, pending, ctx, cache) -> pending``.
``h`` is the 32-bit residual stream, updated in place; ``pending`` is the output of
the previous branch that has not been added to ``h`` yet (or ``None``), so that the
addition can be fused with the next norm, as the reference does after attention and
after the feed-forward (src/model.cu:961-968, 1006-1018).

``prenorm``: ``h += pending; a = mixer(norm1(h)); h += a; pending = ffn(norm2(h))``.
"""
from __future__ import annotations

from .base import register_part


@register_part("arrangement", "prenorm")
def run_prenorm(layer, h, pending, ctx, cache):
    n = layer.mixer_norm.forward(h, pending)
    a = layer.mixer.forward(n, ctx, cache)
    n = layer.feed_forward_norm.forward(h, a)
    return layer.feed_forward.forward(n, ctx)
