"""RMSNorm, fused with the residual addition that precedes it.

``forward(h, delta)`` performs ``h ← h + delta`` in place on the 32-bit residual
stream and returns ``norm(h)`` in the compute dtype, which is the reference's fused
kernel (src/kernels/elementwise.cu:463-506; the plain norm is :30-72).  The weight
multiplies directly (no ``1 + w``) and all arithmetic is 32-bit.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: ``eps``; ``name`` (tensor name relative to the prefix)."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        return {"weight": (params["name"], WeightSpec((hidden_size,), init=(1.0, 0.02)))}

    def load(self, tensors):
        self.weight = self._vector32(tensors["weight"])
        self.eps = float(self.params["eps"])

    def rms_params(self):
        """(weight, eps): offered so that a kernel may apply this norm in its own prologue.  A
        norm that offers it promises that its ``forward`` is exactly this RMSNorm."""
        return self.weight, self.eps

    def forward(self, h, delta=None, rows=None, write_h=True):
        R = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((R, h.shape[1]), dtype=self.dtype, device=h.device)
        ops.add_rmsnorm(h, delta, self.weight, out, self.eps, rows=rows,
                        write_h=write_h and rows is None and delta is not None)
        return out

    def weight_bytes(self):
        return self.weight.numel() * 4
