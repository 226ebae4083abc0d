"""Arrangements: how a layer's branches are wired to the residual stream.

An arrangement is a function ``run(layer, h, pending, ctx, caches) -> pending``.
``h`` is the 32-bit residual stream, updated in place; ``pending`` is the output of
the previous branch that has not been added to ``h`` yet (or ``None``), so that the
addition can be fused with the next norm, as the reference does after attention and
after the feed-forward (src/model.cu:961-968, 1006-1018).  ``layer.branches`` is the
ordered list of the layer's branches (role, part, norm before it, norm after it) and
``caches[k]`` is what branch ``k`` keeps between steps (or ``None``).

``residual``: one branch after the other, ``h += post_norm(part(norm(h)))`` each.  With a
mixer and a feed-forward behind a norm each this is the reference's block.

A part may offer ``forward_from_residual(h, norm, ctx[, cache]) -> bool``: it then reads
the residual stream itself, applies the given norm inside its first kernel and adds its
output into ``h`` inside its last one (the fused few-token kernels do this).  It returns
False when it cannot take the step, and the arrangement falls back to the separate norm
and the returned branch.  Parts without the method just use that path.
"""
from __future__ import annotations

from .base import register_part


def call_part(branch, x, ctx, cache):
    """A mixer sees the step and its cache, a feed-forward only the step."""
    if branch.role == "mixer":
        return branch.part.forward(x, ctx, cache)
    return branch.part.forward(x, ctx)


@register_part("arrangement", "residual")
def run_residual(layer, h, pending, ctx, caches):
    for branch, cache in zip(layer.branches, caches):
        part = branch.part
        if (pending is None and branch.norm is not None and branch.post_norm is None
                and hasattr(part, "forward_from_residual")):
            took = (part.forward_from_residual(h, branch.norm, ctx, cache)
                    if branch.role == "mixer" else part.forward_from_residual(h, branch.norm, ctx))
            if took:
                continue
        if branch.norm is not None:
            x = branch.norm.forward(h, pending)              # h += pending; x = norm(h)
            pending = None
        else:
            if pending is not None:
                h.add_(pending)
                pending = None
            x = h.to(part.dtype)
        y = call_part(branch, x, ctx, cache)
        if branch.post_norm is not None:
            y = branch.post_norm.forward(y.to(h.dtype).contiguous())
        pending = y
    return pending


# the name the two-branch block had before blocks became lists of branches
register_part("arrangement", "prenorm")(run_residual)
