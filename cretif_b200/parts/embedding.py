"""Token embedding and the output head.

The embedding gathers rows of ``[vocab, hidden]`` without scaling
(src/embedding.cu:39-60) into the 32-bit residual stream; the head multiplies the
normed rows that were asked for by ``[vocab, hidden]ᵀ`` (src/embedding.cu:85-135),
sharing the embedding matrix when the model ties them (src/model.cu:1024-1039).
The reference computes logits for every row of a step; the head here only sees the
rows whose logits are wanted.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """params: ``name``; sized by the model's vocabulary (``vocab_size`` is injected)."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        return {"table": (params["name"], WeightSpec((params["vocab_size"], hidden_size)))}

    def load(self, tensors):
        self.table = self._matrix(tensors["table"])

    def forward(self, ids, ctx):
        h = torch.empty((ids.numel(), self.hidden_size), dtype=torch.float32, device=ids.device)
        ops.embed_rows(self.table, ids, h, ctx.fault)
        return h

    def weight_bytes(self):
        return self.table.numel() * self.table.element_size()


@register_part("head", "linear_head")
class LinearHead(Part):
    """params: ``tied`` (share the embedding matrix), ``name``, ``vocab_size``."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        if params.get("tied"):
            return {}
        return {"weight": (params["name"], WeightSpec((params["vocab_size"], hidden_size)))}

    def load(self, tensors):
        self.weight = None if self.params.get("tied") else self._matrix(tensors["weight"])

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.table

    def forward(self, n, ctx):
        return linear(n, self.weight, out_dtype=torch.float32)

    def forward_from_residual(self, h, pending, norm, rows, ctx):
        """Few wanted rows, bfloat16: final norm and head product in one kernel; None if the
        step does not qualify."""
        from .attention import FUSED_MAX_TOKENS, fused_steps_enabled
        R = h.shape[0] if rows is None else rows.numel()
        rms = getattr(norm, "rms_params", None)
        if (pending is not None or not fused_steps_enabled() or self.dtype != torch.bfloat16
                or R > FUSED_MAX_TOKENS or rms is None
                or not ops.fused_supported(R, self.hidden_size, self.weight)):
            return None
        logits = torch.empty((R, self.weight.shape[0]), dtype=torch.float32, device=h.device)
        norm_w, eps = rms()
        ops.fused_norm_linear(h, norm_w, eps, self.weight, logits, rows=rows)
        return logits

    def weight_bytes(self):
        if self.params.get("tied") or self.weight is None:
            return 0
        return self.weight.numel() * self.weight.element_size()
