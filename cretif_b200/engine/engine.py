"""The engine: a loaded model, its cache, and the one step function.

``Engine.step`` takes a batch of sequences, each with its next tokens — a whole
prompt, a further chunk of one, or a single decoded token, in any mixture — runs
exactly the tokens it is given against what earlier steps left in the cache, and
returns the logits at the places that were asked for.  Nothing is padded: tokens of
all sequences are packed one sequence after another, so padding cannot change a
result.  A step in which every sequence brings one token takes the decode kernels;
any other step takes the kernels for ragged prompts, which start each sequence at the
position its cache has reached.

The reference's step is ``TransformerModel::forward(token_ids)`` for one sequence
with an implicit position: any number of tokens at any cached position, the causal
mask offset by what is cached (src/model.cu:831-1040, src/attention.cu:60-77, 695);
its checks (empty input, overflow of the context, src/model.cu:832-849) are made here
on the host before anything is launched.

There is one way through a step — :meth:`Engine.context` builds what the parts read,
:meth:`Engine.run` brackets the launch with the cache's bookkeeping — and both
``Engine.step`` and the generation loop's decode graph go that way.
"""
from __future__ import annotations

import array
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
    """A step that cannot be run as asked (bad tokens, unknown slot), or whose kernels
    reported a fault."""


def _ids_array(tokens) -> np.ndarray:
    """A sequence's token ids as a flat int64 array.  A plain list of Python ints, what
    ``generate`` is given, goes through ``array.array``, which packs it in about half the time
    ``numpy.asarray`` takes (16,384 ids: 0.29 against 0.49 ms)."""
    if type(tokens) is list:
        try:
            return np.frombuffer(array.array("q", tokens), dtype=np.int64)
        except (TypeError, OverflowError):
            pass
    return np.asarray(tokens, dtype=np.int64).reshape(-1)


class _PinnedRing:
    """Page-locked staging buffers for the small host-to-device copies of a step, reused in
    turn; a buffer is taken again only after the copy that last read it has finished."""

    def __init__(self, n: int = 8, n_large: int = 2, large: int = 1 << 14):
        # the last `n_large` buffers take the copies of more than `large` elements (a prompt
        # step's indices): page-locking megabytes costs milliseconds, and such steps do not
        # run ahead of one another, so two buffers serve them
        self.bufs = [None] * (n + n_large)
        self.events = [None] * (n + n_large)
        self.n, self.n_large, self.large = n, n_large, large
        self.at = 0
        self.at_large = 0

    def copy_to(self, dst: torch.Tensor, src: np.ndarray) -> None:
        if src.size > self.large:
            i = self.n + self.at_large
            self.at_large = (self.at_large + 1) % self.n_large
        else:
            i = self.at
            self.at = (i + 1) % self.n
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        if buf is None or buf.numel() < src.size:
            buf = self.bufs[i] = torch.empty(max(1024, 2 * src.size), dtype=torch.int32
                                             ).pin_memory()
        buf[:src.size].numpy()[:] = src
        dst[:src.size].copy_(buf[:src.size], non_blocking=True)
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()


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
        self.fault = ops.fault_word(self.device)
        self.vocab_size = self.spec.vocab_size
        # Steps whose shape (tokens per sequence, wanted places) repeats are captured as CUDA
        # graphs on their second appearance and replayed afterwards; the least recently used
        # ones are dropped.  Indices, slots and positions are read from a fixed device buffer
        # that is refreshed before each replay, so a captured step serves any sequences.
        self.step_graphs = step_graphs and self.model.graph_safe
        self.graph_max_tokens = 32768                # a captured step pins its activations
        self.graph_max_logit_bytes = 128 << 20       # a captured step pins its logits
        self.max_step_graphs = 16
        self._graphs = collections.OrderedDict()
        self._seen: Dict[tuple, int] = {}
        self._last_meta_len = 0
        self._graph_stream = torch.cuda.Stream(device=self.device)
        self._graph_pool = torch.cuda.graph_pool_handle()
        self._staging = _PinnedRing()

    # -- slots -------------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # -- the step ------------------------------------------------------------------
    def context_bucket(self, context: int) -> int:
        """The context length a decode step is planned for: the next power of two (from 512)
        at or above the longest live context, capped by the longest sequence allowed.  The
        split of the keys among CTAs depends on it, so steps of one bucket can share a
        captured graph and a step is planned the same way whether it is captured or not."""
        b = 512
        while b < context:
            b *= 2
        return min(b, self.cache.max_len)

    def context(self, *, T, B, tok_ids, tok_pos, tok_seq, seq_slot, seq_start, cu_seqlens,
                is_decode, max_new, max_context, slots=(), starts=(), news=()) -> StepContext:
        """The one place a StepContext is made (index tensors on the device, int32)."""
        if is_decode:
            max_context = self.context_bucket(max_context)
        return StepContext(
            T=T, B=B, tok_ids=tok_ids, tok_pos=tok_pos, tok_seq=tok_seq, seq_slot=seq_slot,
            seq_start=seq_start, cu_seqlens=cu_seqlens, is_decode=is_decode, max_new=max_new,
            max_context=max_context, fault=self.fault, dtype=self.dtype, device=self.device,
            seq_slot_host=tuple(slots), seq_start_host=tuple(starts), seq_new_host=tuple(news))

    def run(self, pairs, launch):
        """The one way a step runs: the cache makes room for ``pairs`` (slot, new tokens),
        ``launch()`` puts the step's kernels on the stream, the cache counts the tokens."""
        self.cache.begin_step(pairs)
        out = launch()
        self.cache.end_step(pairs)
        return out

    def make_context(self, entries: Sequence[Entry], want, meta: Optional[torch.Tensor] = None
                     ) -> Tuple[StepContext, torch.Tensor, int]:
        """Validate a step on the host and put its index arrays on the device (into ``meta``
        when a buffer of the right size is given, else into a new tensor)."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        toks = [_ids_array(t) for _, t in entries]
        new = np.array([t.size for t in toks], dtype=np.int64)
        if (new == 0).any():
            raise StepError("every sequence of a step must bring at least one token")
        starts = np.array([self.cache.length(s) for s in slots], dtype=np.int64)
        ids = np.concatenate(toks)
        if ids.min() < 0 or ids.max() >= self.vocab_size:
            bad = int(ids[(ids < 0) | (ids >= self.vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary [0, {self.vocab_size})")
        B, T = len(entries), int(new.sum())
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(new, out=cu[1:])
        tok_seq = np.repeat(np.arange(B), new)
        tok_pos = np.arange(T) - cu[tok_seq] + starts[tok_seq]
        if isinstance(want, str) and want == "last":
            rows = cu[1:] - 1
        elif isinstance(want, str) and want == "all":
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
        if meta is None:
            meta = torch.empty(packed.size, dtype=torch.int32, device=self.device)
        self._staging.copy_to(meta, packed)
        o = 0

        def take(n):
            nonlocal o
            out = meta[o:o + n]
            o += n
            return out
        ctx = self.context(
            T=T, B=B, tok_ids=take(T), tok_pos=take(T), tok_seq=take(T), seq_slot=take(B),
            seq_start=take(B), cu_seqlens=take(B + 1), is_decode=bool((new == 1).all()),
            max_new=int(new.max()), max_context=int((starts + new).max()), slots=slots,
            starts=(int(s) for s in starts), news=(int(n) for n in new))
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

            def launch():
                captured["graph"].replay()
                return captured["logits"].clone()
            self._graphs.move_to_end(key)
        else:
            ctx, want_rows, n_want = self.make_context(entries, want)

            def launch():
                return self.model.forward(ctx, self.cache, None if all_rows else want_rows)
        pairs = list(zip(ctx.seq_slot_host, ctx.seq_new_host))
        logits = self.run(pairs, launch)
        if captured is None and key is not None:
            self._maybe_capture(key, entries, want, all_rows, ctx, n_want)
        if check:
            self.check_fault()
        return logits

    # -- captured steps --------------------------------------------------------------
    def _shape_key(self, entries, want):
        """What a captured step depends on beyond the indices it reads from the device: how
        many tokens each sequence brings, where logits are wanted, and for a decode step the
        context length it is planned for."""
        news = tuple(len(t) for _, t in entries)
        if sum(news) > self.graph_max_tokens:
            return None
        w = want if isinstance(want, str) else tuple(tuple(int(i) for i in x) for x in want)
        bucket = 0
        if all(n == 1 for n in news):
            longest = max((int(self.cache.lengths[int(s)]) for s, _ in entries), default=0) + 1
            bucket = self.context_bucket(longest)
        return (news, w, bucket)

    def _maybe_capture(self, key, entries, want, all_rows, ran: StepContext, n_want) -> None:
        """A step shape seen for the second time is captured as a CUDA graph.  The step that
        was just run left the cache as the capture expects it (the capture launches nothing),
        so the capture's context is the finished step's, rebuilt on a buffer of its own."""
        if n_want * self.vocab_size * 4 > self.graph_max_logit_bytes:
            return
        self._seen[key] = self._seen.get(key, 0) + 1
        if self._seen[key] < 2:
            return
        if len(self._seen) > 4096:
            self._seen.clear()
        meta = torch.zeros(self._last_meta_len, dtype=torch.int32, device=self.device)
        saved = {s: int(self.cache.lengths[s]) for s in ran.seq_slot_host}
        for s, n in zip(ran.seq_slot_host, ran.seq_new_host):
            self.cache.lengths[s] -= n              # as they were when the step began
        try:
            ctx, want_rows, _ = self.make_context(entries, want, meta=meta)
        finally:
            for s, n in saved.items():
                self.cache.lengths[s] = n
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
