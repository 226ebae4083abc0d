"""Arrangements: how a layer's norms, mixer and feed-forward are wired.

An arrangement is a function ``run(layer, h, pending, ctx, cache) -> pending``.
``h`` is the 32-bit residual stream, updated in place; ``pending`` is the output of
the previous branch that has not been added to ``h`` yet (or ``None``), so that the
addition can be fused with the next norm, as the reference does after attention and
after the feed-forward (src/model.cu:961-968, 1006-1018).

``prenorm``: ``h += pending; a = mixer(norm1(h)); h += a; pending = ffn(norm2(h))``.

A mixer or feed-forward may offer ``forward_from_residual(h, norm, ctx[, cache]) -> bool``:
it then reads the residual stream itself, applies the given norm inside its first kernel and
adds its output into ``h`` inside its last one (the fused decode kernels do this for steps of
few tokens).  It returns False when it cannot take the step, and the arrangement falls back
to the separate norm and the returned branch.  Parts without the method just use that path.
"""
from __future__ import annotations

from .base import register_part


@register_part("arrangement", "prenorm")
def run_prenorm(layer, h, pending, ctx, cache):
    mixer, ff = layer.mixer, layer.feed_forward
    a = None
    if not (pending is None and hasattr(mixer, "forward_from_residual")
            and mixer.forward_from_residual(h, layer.mixer_norm, ctx, cache)):
        n = layer.mixer_norm.forward(h, pending)
        a = mixer.forward(n, ctx, cache)
    if (a is None and hasattr(ff, "forward_from_residual")
            and ff.forward_from_residual(h, layer.feed_forward_norm, ctx)):
        return None
    n = layer.feed_forward_norm.forward(h, a)
    return ff.forward(n, ctx)
