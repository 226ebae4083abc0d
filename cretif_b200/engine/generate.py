"""The generation loop: batches of unequal prompts, stop tokens, sequences that end
earlier, and as many batches one after another as there are requests.

The loop's decisions are kept apart from the GPU: :class:`GenerationLoop` talks to a
*backend* with five methods (``start_batch``, ``prefill``, ``decode``, ``release``,
``end_batch``), so the decisions can be tested with a scripted backend on the CPU.
:class:`EngineBackend` is the real one.

Behaviour follows the reference's loop (src/model.cu:1046-1100): the whole prompt is
run in one step and the first token is sampled from its last position; then one token
per step; a sampled stop id ends the sequence and is kept in the output (:1082 tests
the id before feeding it); ``max_tokens`` counts sampled tokens including the first
(:1081).  Where the reference throws when the context overflows (:843-849), a
sequence here ends with reason ``"length"`` when its cache is full.
"""
from __future__ import annotations

import collections
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from ..sampling import Sampler, SamplingParams


@dataclass
class GenerationResult:
    prompt_len: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None        # "stop" or "length"


MAX_BACKENDS = 4      # sets of decode graphs kept per engine (one per temperature / top_k)


class GenerationLoop:
    """Decides what runs when; owns no tensors.

    ``capacity_tokens`` is what the cache can hold at once (sequence lengths rounded up
    to ``block_tokens``), ``max_len`` the longest sequence, ``max_batch`` the most
    sequences that start together.
    """

    def __init__(self, backend, stop_ids: Iterable[int], capacity_tokens: int, max_len: int,
                 block_tokens: int = 64, max_batch: int = 64):
        if max_batch <= 0:
            raise ValueError("max_batch must be positive")
        self.backend = backend
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.capacity_tokens, self.max_len = capacity_tokens, max_len
        self.block_tokens, self.max_batch = block_tokens, max_batch

    def _reserve_len(self, prompt_len: int, max_tokens: int) -> int:
        # the last sampled token is never fed back, so it needs no cache position
        return min(prompt_len + max(max_tokens, 1) - 1, self.max_len)

    def _rounded(self, n: int) -> int:
        return -(-n // self.block_tokens) * self.block_tokens

    def plan_batches(self, prompt_lens: Sequence[int], max_tokens: int) -> List[List[int]]:
        """Cut request indices, in order, into batches the cache can hold."""
        batches: List[List[int]] = []
        cur: List[int] = []
        used = 0
        for i, n in enumerate(prompt_lens):
            if n <= 0:
                raise ValueError(f"request {i}: the prompt is empty")
            if n > self.max_len:
                raise ValueError(f"request {i}: the prompt has {n} tokens, the longest "
                                 f"sequence allowed is {self.max_len}")
            need = self._rounded(self._reserve_len(n, max_tokens))
            if need > self.capacity_tokens:
                raise ValueError(f"request {i} needs {need} cache tokens, the cache holds "
                                 f"{self.capacity_tokens}")
            if cur and (len(cur) >= self.max_batch or used + need > self.capacity_tokens):
                batches.append(cur)
                cur, used = [], 0
            cur.append(i)
            used += need
        if cur:
            batches.append(cur)
        return batches

    def run(self, prompts: Sequence[Sequence[int]], max_tokens: int) -> List[GenerationResult]:
        results = [GenerationResult(prompt_len=len(p)) for p in prompts]
        if max_tokens <= 0:
            for r in results:
                r.finish_reason = "length"
            return results
        for batch in self.plan_batches([len(p) for p in prompts], max_tokens):
            self._run_batch(batch, prompts, max_tokens, results)
        return results

    def _record(self, res: GenerationResult, token: int, max_tokens: int) -> bool:
        """Append a sampled token; True if the sequence is finished."""
        res.tokens.append(int(token))
        if int(token) in self.stop_ids:
            res.finish_reason = "stop"
        elif len(res.tokens) >= max_tokens:
            res.finish_reason = "length"
        elif res.prompt_len + len(res.tokens) > self.max_len:
            res.finish_reason = "length"       # no room to feed this token back
        return res.finish_reason is not None

    def _run_batch(self, batch, prompts, max_tokens, results) -> None:
        be = self.backend
        reserve = [self._reserve_len(len(prompts[i]), max_tokens) for i in batch]
        be.start_batch(batch, [prompts[i] for i in batch], reserve)
        try:
            first = be.prefill()
            active: List[int] = []
            for pos, (i, tok) in enumerate(zip(batch, first)):
                if self._record(results[i], tok, max_tokens):
                    be.release(pos)
                else:
                    active.append(pos)
            while active:
                toks = be.decode(active)
                still: List[int] = []
                for pos, tok in zip(active, toks):
                    if self._record(results[batch[pos]], tok, max_tokens):
                        be.release(pos)
                    else:
                        still.append(pos)
                active = still
        finally:
            be.end_batch()


class DecodeRunner:
    """One decode step of a fixed batch as a CUDA graph: embed the last tokens, run the
    layers, head, sample, then advance ids and positions on the device.  Between two
    launches with the same batch nothing is copied to the device.  The step's context comes
    from ``Engine.context`` and its launch goes through ``Engine.run``, like every step; a
    graph is kept per (batch size, context bucket)."""

    def __init__(self, engine, sampler: Sampler, use_graph: bool = True):
        use_graph = use_graph and engine.model.graph_safe
        self.engine, self.sampler, self.use_graph = engine, sampler, use_graph
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.bufs: Dict[int, dict] = {}
        self.stream = torch.cuda.Stream(device=engine.device)
        self.pool = torch.cuda.graph_pool_handle() if use_graph else None

    def _buffers(self, B: int) -> dict:
        if B not in self.bufs:
            dev = self.engine.device
            ints = torch.zeros(6 * B + 1, dtype=torch.int32, device=dev)
            b = {"ints": ints, "tok_ids": ints[0:B], "tok_pos": ints[B:2 * B],
                 "seq_slot": ints[2 * B:3 * B], "seq_start": ints[3 * B:4 * B],
                 "draw": ints[4 * B:5 * B], "sampled": ints[5 * B:6 * B],
                 "tok_seq": torch.arange(B, dtype=torch.int32, device=dev),
                 "cu": torch.arange(B + 1, dtype=torch.int32, device=dev),
                 "request": torch.zeros(B, dtype=torch.int64, device=dev),
                 "logits": None}
            self.bufs[B] = b
        return self.bufs[B]

    def load(self, slots, tokens, positions, requests, draws) -> None:
        """Put a batch's state on the device (called when the batch's make-up changes)."""
        B = len(slots)
        b = self._buffers(B)
        packed = np.concatenate([tokens, positions, slots, positions, draws,
                                 np.zeros(B + 1, dtype=np.int64)]).astype(np.int32)
        b["ints"].copy_(torch.from_numpy(packed).pin_memory(), non_blocking=True)
        b["request"].copy_(torch.from_numpy(np.asarray(requests, dtype=np.int64)).pin_memory(),
                           non_blocking=True)
        self.B = B

    def _body(self, b: dict, B: int, context: int) -> None:
        eng = self.engine
        ctx = eng.context(T=B, B=B, tok_ids=b["tok_ids"], tok_pos=b["tok_pos"],
                          tok_seq=b["tok_seq"], seq_slot=b["seq_slot"],
                          seq_start=b["seq_start"], cu_seqlens=b["cu"], is_decode=True,
                          max_new=1, max_context=context)
        logits = eng.model.forward(ctx, eng.cache, None)
        b["logits"] = logits
        self.sampler(logits, b["sampled"], b["request"], b["draw"])
        ops.advance_decode(b["tok_ids"], b["tok_pos"], b["seq_start"], b["sampled"], B)

    def run(self, context: int) -> torch.Tensor:
        """Launch one step for the loaded batch, whose longest sequence will hold ``context``
        tokens after it; returns the device tensor of sampled ids."""
        B = self.B
        b = self._buffers(B)
        if not self.use_graph:
            self._body(b, B, context)
            return b["sampled"]
        key = (B, self.engine.context_bucket(context))
        if key not in self.graphs:
            # Warm up outside the capture (lazy initialisation, kernel loading), restoring
            # the state the warm-up advanced, then capture.
            saved = b["ints"].clone()
            cur = torch.cuda.current_stream()
            self.stream.wait_stream(cur)
            with torch.cuda.stream(self.stream):
                self._body(b, B, context)
                b["ints"].copy_(saved)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=self.pool, stream=self.stream):
                    self._body(b, B, context)
            cur.wait_stream(self.stream)
            b["ints"].copy_(saved)
            self.graphs[key] = g
        self.graphs[key].replay()
        return b["sampled"]


class EngineBackend:
    """Runs the loop's decisions on an :class:`Engine`.

    Decode steps run ahead of the host: ``decode`` hands the loop the tokens of the oldest
    step in flight and keeps ``depth`` further steps launched, so the device never waits for
    the host to look at tokens, to do the cache's bookkeeping or to launch.  Ids and positions
    advance on the device, so a step needs nothing from the host as long as the batch's
    make-up stays the same.  Which sequences have room for another token is known without
    looking at tokens; what the loop decides from tokens (a stop token) comes one or two steps
    late: that sequence's part of the steps in flight is dropped, its slot is given back
    once they have finished, and before a step with another make-up is launched the steps in
    flight are waited for, because their tokens are that step's input.
    """

    def __init__(self, engine, params: SamplingParams, use_graph: bool = True,
                 run_ahead: bool = True):
        self.engine = engine
        self.sampler = Sampler(params, engine.vocab_size)
        self.runner = DecodeRunner(engine, self.sampler, use_graph)
        self.depth = 2 if run_ahead else 0
        self._loaded: Optional[tuple] = None
        self._queue: List[dict] = []              # launched, oldest first
        self._ready: List[Dict[int, int]] = []    # finished and read, not yet handed out
        self._to_free: List[int] = []

    def start_batch(self, request_ids, prompts, reserve_lens) -> None:
        eng = self.engine
        self.request_ids = list(request_ids)
        self.prompts = [list(p) for p in prompts]
        self.reserve = [int(n) for n in reserve_lens]
        self.slots: List[Optional[int]] = []
        self._queue, self._ready, self._to_free = [], [], []
        # pinned buffers for the sampled ids, one per step that can be in flight
        if len(getattr(self, "_hosts", [[]])[0]) < len(reserve_lens):
            self._hosts = [torch.empty(len(reserve_lens), dtype=torch.int32).pin_memory()
                           for _ in range(self.depth + 2)]
        self._host_at = 0
        try:
            for i, n in enumerate(reserve_lens):
                s = eng.alloc_slot()
                self.slots.append(s)
                eng.cache.reserve(s, n, flush=i + 1 == len(reserve_lens))   # one copy for all
        except Exception:
            self.end_batch()
            raise
        self.last = [0] * len(self.slots)
        self.n_sampled = [0] * len(self.slots)
        self._loaded = None

    def prefill(self) -> List[int]:
        eng = self.engine
        logits = eng.step(list(zip(self.slots, self.prompts)), "last", check=False)
        B = len(self.slots)
        out = torch.empty(B, dtype=torch.int32, device=eng.device)
        req = torch.from_numpy(np.asarray(self.request_ids, dtype=np.int64)).pin_memory().to(
            eng.device, non_blocking=True)
        draw = torch.zeros(B, dtype=torch.int32, device=eng.device)
        self.sampler(logits, out, req, draw)
        toks = out.cpu().tolist()
        eng.check_fault()
        for i, t in enumerate(toks):
            self.last[i], self.n_sampled[i] = t, 1
        return toks

    # -- one step: launch, and (later) collect -----------------------------------------
    def _launch(self, active: Sequence[int]) -> None:
        cache = self.engine.cache
        key = tuple(active)
        slots = np.asarray([self.slots[i] for i in active], dtype=np.int64)
        if key != self._loaded:
            # the state on the device is that of another make-up: this one's comes from the
            # host, which therefore has to have seen every earlier step
            assert not self._queue
            self.runner.load(slots, np.asarray([self.last[i] for i in active]),
                             cache.lengths[slots],
                             np.asarray([self.request_ids[i] for i in active]),
                             np.asarray([self.n_sampled[i] for i in active]))
            self._loaded = key
        entries = [(int(s), 1) for s in slots]
        context = int(cache.lengths[slots].max()) + 1
        sampled = self.engine.run(entries, lambda: self.runner.run(context))
        host = self._hosts[self._host_at][:len(active)]
        self._host_at = (self._host_at + 1) % len(self._hosts)
        host.copy_(sampled, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._queue.append({"active": key, "host": host, "done": done})

    def _collect(self) -> Dict[int, int]:
        """Wait for the oldest step in flight; its tokens by position in the batch."""
        fl = self._queue.pop(0)
        fl["done"].synchronize()
        toks = fl["host"].tolist()
        for i, t in zip(fl["active"], toks):
            self.last[i] = t
            self.n_sampled[i] += 1
        still = [pos for pos in self._to_free if self._in_flight(pos)]
        for pos in self._to_free:            # ended by the loop while steps were running
            if pos not in still:
                self._free(pos)
        self._to_free = still
        return dict(zip(fl["active"], toks))

    def _in_flight(self, pos: int) -> bool:
        return any(pos in fl["active"] for fl in self._queue)

    def _has_room(self, pos: int) -> bool:
        """Whether the next token sampled for ``pos`` can still be fed back (the cache's
        lengths already count the steps in flight)."""
        slot = self.slots[pos]
        return slot is not None and int(self.engine.cache.lengths[slot]) + 1 <= self.reserve[pos]

    def _run_ahead(self, active: Sequence[int]) -> None:
        while len(self._queue) + len(self._ready) < self.depth:
            nxt = tuple(i for i in active if self._has_room(i))
            if not nxt:
                return
            if self._queue and nxt != self._queue[-1]["active"]:
                if any(i not in self._queue[-1]["active"] for i in nxt):
                    return                       # (cannot happen: sequences only ever leave)
                while self._queue:               # another make-up: its input is their output
                    self._ready.append(self._collect())
                continue
            self._launch(nxt)

    def decode(self, active: Sequence[int]) -> List[int]:
        if not self._ready and not self._queue:
            self._launch(active)
        toks = self._ready.pop(0) if self._ready else self._collect()
        out = [toks[i] for i in active]
        if self.depth:
            self._run_ahead(active)
        return out

    def _free(self, pos: int) -> None:
        if self.slots[pos] is not None:
            self.engine.free_slot(self.slots[pos])
            self.slots[pos] = None

    def release(self, pos: int) -> None:
        if self._in_flight(pos):
            if pos not in self._to_free:
                self._to_free.append(pos)    # steps in flight still write to its slot
        else:
            self._free(pos)

    def end_batch(self) -> None:
        try:
            while getattr(self, "_queue", None):
                self._collect()
        except Exception:
            self._queue = []
        self._ready, self._to_free = [], []
        for pos in range(len(self.slots)):
            self._free(pos)
        self._loaded = None
        self.engine.check_fault()


def generate(engine, prompts: Sequence[Sequence[int]], max_tokens: int = 100,
             temperature: float = 0.0, top_k: int = 0, seed: int = 42,
             stop_ids: Optional[Iterable[int]] = None, max_batch: int = 64,
             use_graph: bool = True) -> List[GenerationResult]:
    """Generate up to ``max_tokens`` tokens for every prompt (lists of token ids).

    Option names and defaults are the reference's (``generate(prompt, max_tokens=100,
    temperature=0, top_k=0)``, include/cuinfer/model.h:116-119); ``stop_ids`` defaults
    to the model's ``eos_token_id``.
    """
    params = SamplingParams(float(temperature), int(top_k), int(seed))
    stops = engine.spec.stop_token_ids if stop_ids is None else list(stop_ids)
    # A backend holds the decode graphs; what a graph bakes in is the temperature and top_k
    # (launch constants), not the seed, which the sampling kernel reads from device memory.
    key = (params.temperature, params.top_k, use_graph)
    backends = engine.__dict__.setdefault("_backends", collections.OrderedDict())
    if key not in backends:
        backends[key] = EngineBackend(engine, params, use_graph)
        while len(backends) > MAX_BACKENDS:
            backends.popitem(last=False)
    backends.move_to_end(key)
    backends[key].sampler.set_seed(params.seed)
    loop = GenerationLoop(backends[key], stops, engine.cache.max_tokens, engine.cache.max_len,
                          engine.cache.block_tokens, max_batch)
    return loop.run(prompts, max_tokens)
