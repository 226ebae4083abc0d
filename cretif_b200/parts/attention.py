"""The attention mixer: grouped-query causal attention over the block cache.

Order of work as in the reference's block (src/attention.cu:542-731): q, k, v
projections without bias (:567-576, here one product with the three matrices
stacked), position encoding of q and k (:589-597), cache write (:607-608), scores
scaled after the dot product, causal mask, softmax, weighted sum of values
(:683-714), output projection (:720-728).  Unlike the reference there is no separate
score tensor and no transposition of the cache: the attention kernels read the
cache's blocks directly, for whole prompts and for single tokens alike.
"""
from __future__ import annotations

import torch

from ..cache import KVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, build_part, register_part
from .linear import linear

_force_plain = False
_fused_steps = True
# Steps of at most this many tokens take the fused projection kernels; beyond 32 tokens they
# run as row groups of one launch (measured on a B200: a 64-token step at SmolLM2-135M sizes
# takes half the time of the tensor-core products, whose 128-row tiles run on a few CTAs).
FUSED_MAX_TOKENS = 64


def fused_steps_enabled() -> bool:
    return _fused_steps


def enable_fused_steps(on: bool) -> None:
    """Switch the fused few-token kernels on or off (tests compare both ways)."""
    global _fused_steps
    _fused_steps = bool(on)


def force_plain_attention(on: bool) -> None:
    """Use the one-warp-per-query kernel for every step (the tests' yardstick)."""
    global _force_plain
    _force_plain = bool(on)


@register_part("mixer", "attention")
class Attention(Part):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``, ``window``
    (0 = all keys), ``position`` (a position part's kind and constants), ``names``
    (tensor names of q, k, v, o relative to the layer's prefix)."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.hd = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = int(params.get("window", 0))
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads cannot share {self.nkv} key/value heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ValueError(f"attention: head_dim {self.hd} is not a multiple of 16 in [16, 256]; "
                             "the attention kernels take no other head size")
        pos = dict(params.get("position") or {"kind": "none"})
        self.position = build_part("position", PartSpec(pos.pop("kind"), pos), hidden_size,
                                   dtype, device)
        self.q_dim, self.kv_dim = self.nh * self.hd, self.nkv * self.hd

    @classmethod
    def weight_specs(cls, params, hidden_size):
        q = params["num_heads"] * params["head_dim"]
        kv = params["num_kv_heads"] * params["head_dim"]
        n = params["names"]
        return {"q": (n["q"], WeightSpec((q, hidden_size))),
                "k": (n["k"], WeightSpec((kv, hidden_size))),
                "v": (n["v"], WeightSpec((kv, hidden_size))),
                "o": (n["o"], WeightSpec((hidden_size, q)))}

    def load(self, tensors):
        # one product for q, k and v: rows [q | k | v] of the stacked matrix
        self.w_qkv = self._matrix(torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0))
        self.w_o = self._matrix(tensors["o"])
        self.position.load({})

    def prepare(self, max_positions: int) -> None:
        if hasattr(self.position, "prepare"):
            self.position.prepare(max_positions)

    def cache_request(self):
        return KVRequest(self.nkv, self.hd, self.window)

    def forward(self, x, ctx, cache, into=None):
        """``into``: a float32 matrix that the output is added to (the residual stream) instead
        of being returned."""
        from .linear import plain_forced, skinny_max_rows
        kv = cache.kv
        rot = getattr(self.position, "rotary_table", None)
        rot = rot() if rot is not None else None         # (cos, sin, pairing, rotary_dim)
        o = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=x.device)
        if (self.dtype == torch.bfloat16 and ctx.T > skinny_max_rows() and not plain_forced()
                and not _force_plain and self.hd in (64, 128) and rot is not None
                and rot[3] == self.hd and ops.gemm_tc_supported(x, self.w_qkv, o)):
            # many tokens: rotary and the cache write ride in the product's epilogue
            q = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=x.device)
            ops.gemm_tc_qkv_rope(x, self.w_qkv, q, rot[0], rot[1], rot[2], self.nh,
                                 self.nkv, self.hd, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                                 kv.table, kv.k, kv.v, kv.block_tokens, cache.writes)
            self.attend(q, o, ctx, kv)
        else:
            qkv = linear(x, self.w_qkv)                               # [T, q + 2 kv]
            if rot is not None:          # a rotation by table: one kernel encodes and stores
                ops.rope_kv_append(qkv, rot[0], rot[1], rot[2], rot[3], self.nh, self.nkv,
                                   self.hd, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table,
                                   kv.k, kv.v, kv.block_tokens, cache.writes, ctx.fault)
            else:                        # any other encoding, then the store
                self.position.encode(qkv, ctx, self.nh, self.nkv, self.hd)
                if cache.writes:
                    ops.rope_kv_append(qkv, None, None, 0, 0, self.nh, self.nkv, self.hd,
                                       ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table, kv.k,
                                       kv.v, kv.block_tokens, True, ctx.fault)
            self.attend(qkv, o, ctx, kv)
        if into is not None:
            linear(o, self.w_o, out=into, accumulate=True)
            return None
        return linear(o, self.w_o, out_dtype=torch.float32)

    def forward_from_residual(self, h, norm, ctx, cache) -> bool:
        """bfloat16.  Few tokens: norm + q|k|v + rotary + cache write in one kernel, attention,
        then the output projection added into ``h``.  Many tokens: the same through the norm's
        kernel and the tensor-core products.  False if the step does not qualify."""
        if (ctx.T > FUSED_MAX_TOKENS and self.dtype == torch.bfloat16 and not _force_plain
                and h.dtype == torch.float32 and h.is_contiguous()):
            # many tokens: the norm's own kernel, then the products; the last one adds its
            # float32 accumulators into the residual stream, so that no delta is written, read
            # again and added by the next norm
            self.forward(norm.forward(h, None), ctx, cache, into=h)
            return True
        rms = getattr(norm, "rms_params", None)
        rot = getattr(self.position, "rotary_table", None)
        if (_force_plain or not fused_steps_enabled() or self.dtype != torch.bfloat16
                or ctx.T > FUSED_MAX_TOKENS or rms is None or rot is None or cache is None
                or cache.kv is None or cache.kv.block_tokens & (cache.kv.block_tokens - 1)
                or not ops.fused_supported(ctx.T, self.hidden_size, self.w_qkv)
                or not ops.fused_supported(ctx.T, self.q_dim, self.w_o, norm=False)):
            return False
        cos, sin, pairing, rot_dim = rot()
        if rot_dim != self.hd:
            return False
        norm_w, eps = rms()
        kv = cache.kv
        q = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=h.device)
        ops.fused_qkv_rope(h, norm_w, eps, self.w_qkv, q, cos, sin, pairing, self.nh, self.nkv,
                           self.hd, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table, kv.k, kv.v,
                           kv.block_tokens, cache.writes, ctx.fault)
        o = torch.empty((ctx.T, self.q_dim), dtype=self.dtype, device=h.device)
        self.attend(q, o, ctx, kv)
        ops.fused_linear_add(o, self.w_o, h)
        return True

    def attend(self, q, o, ctx, kv):
        if not _force_plain and self.dtype == torch.bfloat16:
            if ctx.is_decode and ops.attn_decode_supported(self.hd, kv.block_tokens,
                                                           self.nh // self.nkv):
                splits, cluster = ops.decode_plan(ctx.B, self.nkv, ctx.max_context, q.device,
                                                  self.hd)
                ops.attn_decode(q, o, kv.k, kv.v, kv.table, ctx.tok_pos, ctx.tok_seq,
                                ctx.seq_slot, self.nh, self.nkv, self.hd, self.scale,
                                self.window, kv.block_tokens, splits, ctx.fault, cluster)
                return
            if not ctx.is_decode and ops.attn_prefill_supported(self.hd, kv.block_tokens):
                ops.attn_prefill(q, o, kv.k, kv.v, kv.table, ctx.cu_seqlens, ctx.seq_start,
                                 ctx.seq_slot, self.nh, self.nkv, self.hd, self.scale,
                                 self.window, kv.block_tokens, ctx.B, ctx.max_new, ctx.fault)
                return
        ops.attn_simt(q, o, kv.k, kv.v, kv.table, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                      self.nh, self.nkv, self.hd, self.scale, self.window, kv.block_tokens)

    def weight_bytes(self):
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()
