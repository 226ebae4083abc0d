"""The whole-step decode kernel: one persistent launch for embed → all layers → head.

For steps of few tokens in bfloat16 a model whose scheduled layers are all
``rmsnorm → attention(rotary) → rmsnorm → gated_mlp`` in the ``prenorm`` arrangement can be
run by ``csrc/decode_step.cu`` instead of five launches per layer.  This module looks at an
assembled :class:`~cretif_b200.engine.model.Model`, decides whether it qualifies, builds the
per-visit records the kernel reads (weights, norm weights, the visit's cache and its TMA
maps) and launches it.  Parts know nothing of it; a model that does not qualify, a step with
more tokens, float32, or ``enable(False)`` simply take the kernels of the parts.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import ops
from ..parts.attention import Attention
from ..parts.embedding import LinearHead, TokenEmbedding
from ..parts.mlp import GatedMLP
from ..parts.norm import RMSNorm
from ..parts.position import Rotary

# Off by default.  Measured on a B200 at SmolLM2-135M sizes (batch 8, context 2,050): the
# persistent kernel takes 1.15 ms per step against 0.81 ms for the separate fused kernels
# replayed as a graph.  Its phases cost 5.8 / 18.5 / 3.3 / 5.6 / 4.1 µs (q|k|v, attention,
# o-proj, gate|up, down; each including its grid barrier): every phase is a chain of four or
# five dependent L2 round trips whichever way it is launched, the barrier is not cheaper than
# a programmatic dependent launch, and one CTA per SM runs the attention ranges one after
# another.  It stays as a tested alternative (`enable(True)`).
_enabled = False
MAX_TOKENS = 32


def enable(on: bool) -> None:
    """Switch the whole-step kernel on or off (tests compare both ways)."""
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


class StepKernel:
    """Built once per (model, cache); ``run`` replaces ``Model.forward`` for small steps."""

    def __init__(self, model, cache):
        self.model, self.cache = model, cache
        self._checked = False
        self._reason: Optional[str] = None

    # The kernel lives in a library of its own that takes half a minute to compile, so nothing
    # here touches it before somebody switches the kernel on or asks whether the model fits.
    def _ensure(self) -> None:
        if not self._checked:
            self._checked = True
            self._reason = self._qualifies()
            if self._reason is None:
                self._build()

    @property
    def reason(self) -> Optional[str]:
        self._ensure()
        return self._reason

    @property
    def ok(self) -> bool:
        return self.reason is None

    # -- does the model fit the kernel? ------------------------------------------------
    def _qualifies(self) -> Optional[str]:
        m = self.model
        if m.dtype != torch.bfloat16:
            return "not bfloat16"
        if type(m.embedding) is not TokenEmbedding or type(m.head) is not LinearHead \
                or type(m.final_norm) is not RMSNorm:
            return "embedding, final norm or head of another kind"
        first = None
        for entry in m.spec.schedule:
            layer, ls = m.layers[entry.layer], m.spec.layers[entry.layer]
            if ls.arrangement != "prenorm":
                return "arrangement is not prenorm"
            a, f = layer.mixer, layer.feed_forward
            if type(a) is not Attention or type(f) is not GatedMLP \
                    or type(layer.mixer_norm) is not RMSNorm \
                    or type(layer.feed_forward_norm) is not RMSNorm:
                return "a layer has other parts"
            if type(a.position) is not Rotary or a.position.rot_dim != a.hd:
                return "position encoding is not rotary over the whole head"
            key = (a.nh, a.nkv, a.hd, a.scale, a.window, a.position.pairing, a.position.theta,
                   f.inter, f.gu_block)
            if first is None:
                first = key
            elif key != first:
                return "layers differ in their sizes or constants"
        a = m.layers[m.spec.schedule[0].layer].mixer
        if a.nh // a.nkv > 8 or not ops.step_lib().cretif_decode_step_supported(1, a.hd):
            return "head size or group size outside the kernel's range"
        if self.cache.block_tokens != 64:
            return "cache blocks are not 64 tokens"
        if m.spec.hidden_size % 8 or m.layers[0].feed_forward.inter % 8:
            return "widths are not multiples of 8"
        return None

    # -- per-visit records ---------------------------------------------------------------
    def _build(self) -> None:
        m, cache, L = self.model, self.cache, ops.step_lib()
        dev = m.device
        size = L.cretif_step_layer_bytes()
        sched = m.spec.schedule
        host = torch.zeros(len(sched) * size, dtype=torch.uint8).pin_memory()
        base = host.data_ptr()
        self._keep = []
        for i, entry in enumerate(sched):
            layer = m.layers[entry.layer]
            a, f = layer.mixer, layer.feed_forward
            cid = i if entry.cache is None else entry.cache
            kv = cache.kv_view(cid)
            rc = L.cretif_step_layer_fill(
                ctypes.c_void_p(base + i * size), ctypes.c_void_p(a.w_qkv.data_ptr()),
                ctypes.c_void_p(a.w_o.data_ptr()), ctypes.c_void_p(f.w_gate_up.data_ptr()),
                ctypes.c_void_p(f.w_down.data_ptr()),
                ctypes.c_void_p(layer.mixer_norm.weight.data_ptr()),
                ctypes.c_void_p(layer.feed_forward_norm.weight.data_ptr()),
                ctypes.c_float(layer.mixer_norm.eps), ctypes.c_float(layer.feed_forward_norm.eps),
                ctypes.c_void_p(kv.k.data_ptr()), ctypes.c_void_p(kv.v.data_ptr()),
                ctypes.c_longlong(kv.k.shape[0]), a.nkv, a.hd,
                ctypes.c_void_p(kv.table.data_ptr()), kv.table.stride(0),
                int(entry.cache is None))
            if rc != 0:
                self._reason = f"layer record {i} refused (status {rc})"
                return
        self.layers_dev = host.to(dev)
        a = m.layers[sched[0].layer].mixer
        f = m.layers[sched[0].layer].feed_forward
        self.a, self.f = a, f
        self.cos, self.sin = a.position._table
        self.barrier = torch.zeros(2, dtype=torch.int32, device=dev)
        self.ctas = ops.sm_count(dev)
        self._scratch = {}
        self.stamps = None          # set to an int64 tensor [5 * layers + 3] to time the phases

    def _buffers(self, B: int, n_splits: int) -> dict:
        key = (B, n_splits)
        if key not in self._scratch:
            m, a, f, dev = self.model, self.a, self.f, self.model.device
            bf, f32 = torch.bfloat16, torch.float32
            self._scratch[key] = {
                "h": torch.empty((B, m.spec.hidden_size), dtype=f32, device=dev),
                "q": torch.empty((B, a.q_dim), dtype=bf, device=dev),
                "attn": torch.empty((B, a.q_dim), dtype=bf, device=dev),
                "act": torch.empty((B, f.inter), dtype=bf, device=dev),
                "part_o": torch.empty((B, a.nh, n_splits, a.hd), dtype=f32, device=dev),
                "part_ml": torch.empty((B, a.nh, n_splits, 2), dtype=f32, device=dev),
            }
        return self._scratch[key]

    def takes(self, ctx) -> bool:
        return (_enabled and self.ok and ctx.is_decode and ctx.T <= MAX_TOKENS
                and bool(ops.step_lib().cretif_decode_step_supported(ctx.T, self.a.hd)))

    def run(self, ctx, want_rows) -> torch.Tensor:
        """Logits [wanted, vocab] of a decode step (every sequence brings one token)."""
        m, a, f = self.model, self.a, self.f
        B = ctx.T
        n_want = B if want_rows is None else int(want_rows.numel())
        V = m.spec.vocab_size
        logits = torch.empty((n_want, V), dtype=torch.float32, device=m.device)
        if n_want == 0:
            return logits
        items_per_split = max(1, B * a.nkv)
        tiles = max(1, -(-ctx.max_context // 64))
        n_splits = max(1, min(tiles, 64, (2 * self.ctas) // items_per_split))
        buf = self._buffers(B, n_splits)
        counters = ops._decode_counters(m.device, B * a.nkv)
        ints = (ctypes.c_int * 14)(len(m.spec.schedule), B, m.spec.hidden_size, f.inter, a.nh,
                                   a.nkv, a.hd, f.gu_block, a.position.pairing, 64, a.window,
                                   n_splits, V, n_want)
        floats = (ctypes.c_float * 2)(m.final_norm.eps, a.scale)
        P = ctypes.c_void_p
        ptrs = (P * 22)(
            self.layers_dev.data_ptr(), buf["h"].data_ptr(), buf["q"].data_ptr(),
            buf["attn"].data_ptr(), buf["act"].data_ptr(), buf["part_o"].data_ptr(),
            buf["part_ml"].data_ptr(), counters.data_ptr(), ctx.tok_ids.data_ptr(),
            ctx.tok_pos.data_ptr(), ctx.tok_seq.data_ptr(), ctx.seq_slot.data_ptr(),
            self.cos.data_ptr(), self.sin.data_ptr(), m.embedding.table.data_ptr(),
            m.final_norm.weight.data_ptr(), m.head.weight.data_ptr(),
            0 if want_rows is None else want_rows.data_ptr(), logits.data_ptr(),
            self.barrier.data_ptr(), ctx.fault.data_ptr(),
            0 if self.stamps is None else self.stamps.data_ptr())
        ops._check(ops.step_lib().cretif_decode_step(ints, floats, ptrs, self.ctas, ops._stream()),
                   "decode_step")
        return logits
