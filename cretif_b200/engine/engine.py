"""The engine: a loaded model, its cache, and the one step function.

``Engine.step`` takes a batch of sequences that either all begin (whole prompts of
unequal lengths, packed into one pass) or all continue by one token, runs exactly the
tokens it is given against what earlier steps left in the cache, and returns the
logits at the places that were asked for.  Nothing is padded: tokens of all
sequences are packed one sequence after another, so padding cannot change a result.

The reference's step is ``TransformerModel::forward(token_ids)`` for one sequence
with an implicit position (src/model.cu:831-1040); its checks (empty input, overflow
of the context, :832-849) are made here on the host before anything is launched.
"""
from __future__ import annotations

import collections
from typing import Dict, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..cache import SequenceCache
from ..config import load_config
from ..csrc import ops
from ..parts.base import StepContext
from ..weights import load_weights
from .model import Model, manifest

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}

_FAULTS = {1: "a token id outside the vocabulary reached the embedding kernel",
           2: "a bounded wait inside a kernel expired",
           4: "a token's position maps to no cache block"}


class StepError(RuntimeError):
    """A step that cannot be run as asked (bad tokens, unknown slot, mixed batch)."""


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}") from None


def require_cuda(device) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"the engine runs on a CUDA device only, got {dev}")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; the engine has no CPU path")
    major, minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        raise RuntimeError(f"the kernels are built for sm_100a (B200); device {dev} is "
                           f"sm_{major}{minor}")
    return dev


Entry = Tuple[int, Sequence[int]]


class Engine:
    """A model on one GPU with its cache.

    ``max_tokens`` is the most tokens live sequences hold at any time (each rounded up
    to a multiple of ``block_tokens``); it sizes the cache.
    """

    def __init__(self, model_dir: str, dtype="bfloat16", max_tokens: int = 8192,
                 device="cuda:0", block_tokens: int = 64, max_slots: Optional[int] = None,
                 max_len: Optional[int] = None, step_graphs: bool = True):
        self.device = require_cuda(device)
        self.dtype = parse_dtype(dtype)
        self.model_dir = model_dir
        self.architecture, self.config, self.spec = load_config(model_dir)
        names, ignorable = manifest(self.spec)
        tensors = load_weights(model_dir, names, ignorable)
        ops.lib()                                    # build or load the kernels now, loudly
        torch.cuda.set_device(self.device)
        self.model = Model(self.spec, self.dtype, self.device)
        self.model.load(tensors)
        del tensors
        longest = min(max_len or self.spec.max_positions, self.spec.max_positions)
        self.cache = SequenceCache(self.model.cache_requests(), max_tokens, self.dtype,
                                   self.device, block_tokens=block_tokens, max_slots=max_slots,
                                   max_len=longest)
        self.model.prepare(self.cache.max_len)
        from .step_kernel import StepKernel
        self.model.step_kernel = StepKernel(self.model, self.cache)
        self.fault = ops.fault_word(self.device)
        self.vocab_size = self.spec.vocab_size
        # Steps whose shape (tokens per sequence, wanted places) repeats are captured as CUDA
        # graphs on their second appearance and replayed afterwards; the least recently used
        # ones are dropped.  Indices, slots and positions are read from a fixed device buffer
        # that is refreshed before each replay, so a captured step serves any sequences.
        self.step_graphs = step_graphs and self.model.graph_safe
        self.graph_max_tokens = 8192
        self.max_step_graphs = 16
        self._graphs = collections.OrderedDict()
        self._seen: Dict[tuple, int] = {}
        self._last_meta_len = 0
        self._graph_stream = torch.cuda.Stream(device=self.device)
        self._graph_pool = torch.cuda.graph_pool_handle()

    # -- slots -------------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # -- the step ------------------------------------------------------------------
    def make_context(self, entries: Sequence[Entry], want, meta: Optional[torch.Tensor] = None
                     ) -> Tuple[StepContext, torch.Tensor, int]:
        """Validate a step on the host and put its index arrays on the device (into ``meta``
        when a buffer of the right size is given, else into a new tensor)."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        toks = [np.asarray(t, dtype=np.int64).reshape(-1) for _, t in entries]
        new = np.array([t.size for t in toks], dtype=np.int64)
        if (new == 0).any():
            raise StepError("every sequence of a step must bring at least one token")
        starts = np.array([self.cache.length(s) for s in slots], dtype=np.int64)
        all_begin, all_one = bool((starts == 0).all()), bool((new == 1).all())
        if not (all_begin or all_one):
            raise StepError("the sequences of a step must either all start at their first "
                            "token or all go on by one token")
        ids = np.concatenate(toks)
        if ids.min() < 0 or ids.max() >= self.vocab_size:
            bad = int(ids[(ids < 0) | (ids >= self.vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary [0, {self.vocab_size})")
        B, T = len(entries), int(new.sum())
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(new, out=cu[1:])
        tok_seq = np.repeat(np.arange(B), new)
        tok_pos = np.arange(T) - cu[tok_seq] + starts[tok_seq]
        if want == "last":
            rows = cu[1:] - 1
        elif want == "all":
            rows = np.arange(T)
        else:
            if len(want) != B:
                raise StepError("`want` must give a list of places for every sequence")
            parts = []
            for b, w in enumerate(want):
                w = np.asarray(list(w), dtype=np.int64).reshape(-1)
                if w.size and (w.min() < 0 or w.max() >= new[b]):
                    raise StepError(f"sequence {b}: wanted places {w.tolist()} are not among "
                                    f"its {int(new[b])} tokens")
                parts.append(cu[b] + w)
            rows = np.concatenate(parts) if parts else np.zeros(0, dtype=np.int64)
        packed = np.concatenate([ids, tok_pos, tok_seq, np.asarray(slots), starts, cu, rows]
                                ).astype(np.int32)
        self._last_meta_len = int(packed.size)
        pinned = torch.from_numpy(packed).pin_memory()
        if meta is None:
            meta = pinned.to(self.device, non_blocking=True)
        else:                                   # the fixed buffer of a captured step
            meta.copy_(pinned, non_blocking=True)
        o = 0

        def take(n):
            nonlocal o
            out = meta[o:o + n]
            o += n
            return out
        ctx = StepContext(
            T=T, B=B, tok_ids=take(T), tok_pos=take(T), tok_seq=take(T), seq_slot=take(B),
            seq_start=take(B), cu_seqlens=take(B + 1), is_decode=all_one,
            max_new=int(new.max()), max_context=int((starts + new).max()), fault=self.fault,
            dtype=self.dtype, device=self.device, seq_slot_host=tuple(slots),
            seq_start_host=tuple(int(s) for s in starts), seq_new_host=tuple(int(n) for n in new))
        want_rows = take(rows.size)
        return ctx, want_rows, int(rows.size)

    def step(self, entries: Sequence[Entry], want: Union[str, Sequence[Sequence[int]]] = "last",
             check: bool = True) -> torch.Tensor:
        """Run one step; returns float32 logits ``[wanted, vocab]`` on the device, in the
        order of ``entries`` and of each entry's wanted places."""
        all_rows = isinstance(want, str) and want == "all"
        key = self._shape_key(entries, want) if self.step_graphs else None
        captured = self._graphs.get(key) if key is not None else None
        if captured is not None:
            # the same step shape has been captured: refresh its indices, replay its kernels
            ctx, want_rows, n_want = self.make_context(entries, want, meta=captured["meta"])
            pairs = [(s, n) for s, n in zip(ctx.seq_slot_host, ctx.seq_new_host)]
            self.cache.begin_step(pairs)
            captured["graph"].replay()
            logits = captured["logits"].clone()
            self._graphs.move_to_end(key)
        else:
            ctx, want_rows, n_want = self.make_context(entries, want)
            pairs = [(s, n) for s, n in zip(ctx.seq_slot_host, ctx.seq_new_host)]
            self.cache.begin_step(pairs)
            logits = self.model.forward(ctx, self.cache, None if all_rows else want_rows)
            if key is not None:
                self._maybe_capture(key, entries, want, all_rows, ctx.T)
        self.cache.end_step(pairs)
        if check:
            self.check_fault()
        return logits

    # -- captured steps --------------------------------------------------------------
    def _shape_key(self, entries, want):
        """What a captured step depends on beyond the indices it reads from the device: how
        many tokens each sequence brings and where logits are wanted."""
        news = tuple(len(t) for _, t in entries)
        if sum(news) > self.graph_max_tokens:
            return None
        w = want if isinstance(want, str) else tuple(tuple(int(i) for i in x) for x in want)
        return (news, w)

    def _maybe_capture(self, key, entries, want, all_rows, T) -> None:
        """A step shape seen for the second time is captured as a CUDA graph (the step that
        was just run left the cache in the state the capture's warm run expects: the capture
        itself launches nothing)."""
        self._seen[key] = self._seen.get(key, 0) + 1
        if self._seen[key] < 2:
            return
        if len(self._seen) > 4096:
            self._seen.clear()
        n_meta = self._last_meta_len
        meta = torch.zeros(n_meta, dtype=torch.int32, device=self.device)
        ctx, want_rows, _ = self.make_context(entries, want, meta=meta)
        graph = torch.cuda.CUDAGraph()
        cur = torch.cuda.current_stream()
        self._graph_stream.wait_stream(cur)
        with torch.cuda.stream(self._graph_stream):
            with torch.cuda.graph(graph, pool=self._graph_pool, stream=self._graph_stream):
                logits = self.model.forward(ctx, self.cache, None if all_rows else want_rows)
        cur.wait_stream(self._graph_stream)
        self._graphs[key] = {"graph": graph, "meta": meta, "logits": logits}
        while len(self._graphs) > self.max_step_graphs:
            self._graphs.popitem(last=False)

    def check_fault(self) -> None:
        """Read the status word the kernels write (synchronises the device)."""
        word = int(self.fault.item())
        if word:
            self.fault.zero_()
            sk = getattr(self.model, "step_kernel", None)
            if sk is not None and sk.ok:
                sk.barrier.zero_()         # a step that gave up may have left it half counted
            what = [msg for bit, msg in _FAULTS.items() if word & bit]
            raise StepError("device fault: " + "; ".join(what or [f"status {word}"]))

    def generate(self, prompts, max_tokens: int = 100, temperature: float = 0.0, top_k: int = 0,
                 seed: int = 42, stop_ids=None, max_batch: int = 64, use_graph: bool = True):
        """Generate for a list of prompts (lists of token ids); see engine.generate.generate."""
        from .generate import generate
        return generate(self, prompts, max_tokens=max_tokens, temperature=temperature,
                        top_k=top_k, seed=seed, stop_ids=stop_ids, max_batch=max_batch,
                        use_graph=use_graph)

    def stats(self) -> dict:
        return {"weights_bytes": self.model.weight_bytes(), "cache": self.cache.stats(),
                "dtype": str(self.dtype).replace("torch.", ""),
                "architecture": self.spec.architecture}
