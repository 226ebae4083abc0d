"""The gated feed-forward (SwiGLU): ``down(act(gate(x)) ⊙ up(x))`` without bias.

Reference: two products, SiLU, multiply, one product (src/ffn.cu:132-191;
``silu(z) = z / (1 + exp(−z))``, src/kernels/elementwise.cu:93-99).  Here gate and up
are one product with the two matrices stacked, and SiLU·mul is one kernel.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear, plain_forced, skinny_max_rows as SKINNY_ROWS


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """params: ``intermediate_size``, ``activation`` ("silu"), ``names`` (gate, up, down)."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.inter = int(params["intermediate_size"])
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: activation {params['activation']!r} has no kernel "
                             "(only 'silu')")

    @classmethod
    def weight_specs(cls, params, hidden_size):
        I, n = params["intermediate_size"], params["names"]
        return {"gate": (n["gate"], WeightSpec((I, hidden_size))),
                "up": (n["up"], WeightSpec((I, hidden_size))),
                "down": (n["down"], WeightSpec((hidden_size, I)))}

    # Rows of the stacked gate|up matrix alternate in groups of this many (64 gate rows, then
    # their 64 up rows) when the tensor-core product can fuse SiLU·mul into its epilogue.
    GU_BLOCK = 64

    def load(self, tensors):
        gate, up = tensors["gate"], tensors["up"]
        I = self.inter
        self.gu_block = self.GU_BLOCK if (self.dtype == torch.bfloat16 and I % self.GU_BLOCK == 0) else 0
        if self.gu_block:
            b = self.gu_block
            stacked = torch.stack([gate.reshape(I // b, b, -1), up.reshape(I // b, b, -1)], dim=1)
            self.w_gate_up = self._matrix(stacked.reshape(2 * I, -1))
        else:
            self.w_gate_up = self._matrix(torch.cat([gate, up], dim=0))
        self.w_down = self._matrix(tensors["down"])

    def forward(self, x, ctx, into=None):
        """``into``: a float32 matrix that the output is added to (the residual stream) instead
        of being returned."""
        T = x.shape[0]
        act = torch.empty((T, self.inter), dtype=self.dtype, device=x.device)
        if (self.gu_block == 64 and T > SKINNY_ROWS() and not plain_forced()
                and ops.gemm_tc_supported(x, self.w_gate_up, act)):
            ops.gemm_tc_silu(x, self.w_gate_up, act)                  # product + SiLU·mul
        else:
            gu = linear(x, self.w_gate_up)                            # [T, 2 I]
            ops.silu_mul(gu, act, self.gu_block)
        if into is not None:
            linear(act, self.w_down, out=into, accumulate=True)
            return None
        return linear(act, self.w_down, out_dtype=torch.float32)

    def forward_from_residual(self, h, norm, ctx) -> bool:
        """bfloat16.  Few tokens: norm + gate|up + SiLU·mul in one kernel, then the down
        projection added into ``h``.  Many tokens: the same through the norm's kernel and the
        tensor-core products.  False if the step does not qualify."""
        from .attention import FUSED_MAX_TOKENS, fused_steps_enabled
        T = h.shape[0]
        if (T > FUSED_MAX_TOKENS and self.dtype == torch.bfloat16 and not plain_forced()
                and h.dtype == torch.float32 and h.is_contiguous()):
            # many tokens: the down projection adds its accumulators into the residual stream
            self.forward(norm.forward(h, None), ctx, into=h)
            return True
        rms = getattr(norm, "rms_params", None)
        if (not fused_steps_enabled() or self.dtype != torch.bfloat16 or T > FUSED_MAX_TOKENS
                or rms is None
                or not ops.fused_supported(T, self.hidden_size, self.w_gate_up)
                or not ops.fused_supported(T, self.inter, self.w_down, norm=False)):
            return False
        act = torch.empty((T, self.inter), dtype=self.dtype, device=h.device)
        norm_w, eps = rms()
        ops.fused_gate_up_silu(h, norm_w, eps, self.w_gate_up, act, self.gu_block)
        ops.fused_linear_add(act, self.w_down, h)
        return True

    def weight_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()
