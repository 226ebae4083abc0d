"""The cache of a model: one slot per sequence, storage per group of layers.

What a layer's mixer keeps between steps is its own business; it tells the
cache by returning a request from ``cache_request()``:

* :class:`KVRequest` — keys and values that grow with the sequence (all of
  them, or a sliding window of the last ``window``);
* :class:`StateRequest` — a tensor of fixed size per sequence;
* ``None`` — nothing.

Requests with the same needs are grouped and each group has storage of its own:
``K, V [layers_in_group, n_blocks, num_kv_heads, block_tokens, head_dim]`` cut
into blocks of ``block_tokens`` positions, a pool of blocks, and a block table
``[max_slots, blocks_per_sequence]`` (int32, mirrored on the device) that maps a
sequence's positions to blocks.  One (block, kv head) tile is contiguous
(``block_tokens × head_dim``), which is what an attention kernel streams.

The reference keeps ``[layers][max_seq][kv_heads][head_dim]`` for one sequence
with one shared length (include/cuinfer/kv_cache.h:57-70, src/kv_cache.cu:42-53,
201-212) and throws on overflow (:167-174); the checks here are made on the host
before anything is launched, in the same spirit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .blocks import BlockPool, CacheError, CacheFull, SlotSet


@dataclass(frozen=True)
class KVRequest:
    num_kv_heads: int
    head_dim: int
    window: int = 0          # 0: every key is kept; W > 0: the last W keys


@dataclass(frozen=True)
class StateRequest:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class KVView:
    """What a mixer gets for one cache id: its layer's slice of the group's storage."""

    k: torch.Tensor              # [n_blocks, num_kv_heads, block_tokens, head_dim]
    v: torch.Tensor
    table: torch.Tensor          # [max_slots, blocks_per_sequence] int32, device
    block_tokens: int
    window: int


class _KVGroup:
    def __init__(self, request: KVRequest, cache_ids: List[int], n_blocks: int,
                 block_tokens: int, max_slots: int, blocks_per_seq: int, dtype, device):
        self.request = request
        self.cache_ids = list(cache_ids)
        self.block_tokens = block_tokens
        self.blocks_per_seq = blocks_per_seq
        shape = (len(cache_ids), n_blocks, request.num_kv_heads, block_tokens, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pool = BlockPool(n_blocks)
        self.table_host = np.full((max_slots, blocks_per_seq), -1, dtype=np.int32)
        self.table = torch.full((max_slots, blocks_per_seq), -1, dtype=torch.int32, device=device)
        self.first_block = np.zeros(max_slots, dtype=np.int64)   # blocks below were released
        self.n_blocks_of = np.zeros(max_slots, dtype=np.int64)   # logical blocks ever mapped
        self.dirty: set = set()

    def blocks_needed(self, slot: int, new_len: int) -> int:
        want = -(-new_len // self.block_tokens)
        return max(0, want - int(self.n_blocks_of[slot]))

    def grow(self, slot: int, new_len: int) -> None:
        n = self.blocks_needed(slot, new_len)
        if n == 0:
            return
        got = self.pool.take(n)
        at = int(self.n_blocks_of[slot])
        self.table_host[slot, at:at + n] = got
        self.n_blocks_of[slot] = at + n
        self.dirty.add(slot)

    def shrink_to(self, slot: int, old_blocks: int) -> None:
        """Undo a grow (used when a later group cannot satisfy the same step)."""
        at = int(self.n_blocks_of[slot])
        if at > old_blocks:
            self.pool.give_back(self.table_host[slot, old_blocks:at].tolist())
            self.table_host[slot, old_blocks:at] = -1
            self.n_blocks_of[slot] = old_blocks
            self.dirty.add(slot)

    def release_outside_window(self, slot: int, length: int) -> None:
        w = self.request.window
        if w <= 0:
            return
        first_needed_key = max(0, length - w + 1)       # the next query sits at `length`
        keep_from = first_needed_key // self.block_tokens
        lo = int(self.first_block[slot])
        if keep_from > lo:
            self.pool.give_back(self.table_host[slot, lo:keep_from].tolist())
            self.table_host[slot, lo:keep_from] = -1
            self.first_block[slot] = keep_from
            self.dirty.add(slot)

    def release_all(self, slot: int) -> None:
        lo, hi = int(self.first_block[slot]), int(self.n_blocks_of[slot])
        if hi > lo:
            self.pool.give_back(self.table_host[slot, lo:hi].tolist())
        self.table_host[slot, :] = -1
        self.first_block[slot] = 0
        self.n_blocks_of[slot] = 0
        self.dirty.add(slot)

    def flush(self) -> None:
        if not self.dirty:
            return
        rows = sorted(self.dirty)
        idx = torch.as_tensor(rows, dtype=torch.int64)
        src = torch.from_numpy(self.table_host[rows])
        if self.table.device.type == "cuda":
            src = src.pin_memory().to(self.table.device, non_blocking=True)
            idx = idx.pin_memory().to(self.table.device, non_blocking=True)
        self.table.index_copy_(0, idx, src)
        self.dirty.clear()


class SequenceCache:
    """Slots, lengths, block tables and storage for all cache ids of a model.

    ``requests`` maps a cache id (the index of the schedule entry that owns the
    cache) to what its mixer asked for.  ``max_tokens`` sizes every key/value
    group: it is the most tokens that live sequences may hold at any time, each
    sequence's count rounded up to a multiple of ``block_tokens``.
    """

    def __init__(self, requests: Dict[int, object], max_tokens: int, dtype: torch.dtype,
                 device, block_tokens: int = 64, max_slots: Optional[int] = None,
                 max_len: Optional[int] = None):
        if block_tokens <= 0 or block_tokens % 16:
            raise ValueError("block_tokens must be a positive multiple of 16")
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        self.block_tokens = block_tokens
        self.n_blocks = -(-max_tokens // block_tokens)
        self.max_tokens = self.n_blocks * block_tokens
        self.max_len = min(max_len or self.max_tokens, self.max_tokens)
        self.blocks_per_seq = -(-self.max_len // block_tokens)
        self.max_slots = max_slots or max(1, min(self.n_blocks, 1024))
        self.dtype, self.device = dtype, torch.device(device)
        self.slots = SlotSet(self.max_slots)
        self.lengths = np.zeros(self.max_slots, dtype=np.int64)

        self._kv_groups: List[_KVGroup] = []
        self._kv_of: Dict[int, Tuple[_KVGroup, int]] = {}
        self._state: Dict[int, torch.Tensor] = {}
        by_request: Dict[KVRequest, List[int]] = {}
        for cid in sorted(requests):
            req = requests[cid]
            if req is None:
                continue
            if isinstance(req, KVRequest):
                by_request.setdefault(req, []).append(cid)
            elif isinstance(req, StateRequest):
                self._state[cid] = torch.zeros((self.max_slots, *req.shape), dtype=req.dtype,
                                               device=self.device)
            else:
                raise TypeError(f"cache id {cid}: unknown cache request {req!r}")
        for req, cids in by_request.items():
            g = _KVGroup(req, cids, self.n_blocks, block_tokens, self.max_slots,
                         self.blocks_per_seq, dtype, self.device)
            self._kv_groups.append(g)
            for i, cid in enumerate(cids):
                self._kv_of[cid] = (g, i)

    # -- slots ---------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        for t in self._state.values():
            t[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.give_back(slot)          # raises on unknown or double free
        for g in self._kv_groups:
            g.release_all(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not in use")
        return int(self.lengths[slot])

    # -- a step ----------------------------------------------------------------
    def begin_step(self, entries: Sequence[Tuple[int, int]]) -> None:
        """Make room for ``n_new`` more tokens in each ``(slot, n_new)``; all or nothing."""
        seen = set()
        for slot, n_new in entries:
            if not self.slots.is_live(slot):
                raise CacheError(f"slot {slot} is not in use")
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n_new <= 0:
                raise CacheError(f"slot {slot}: a step must bring at least one token")
            if self.lengths[slot] + n_new > self.max_len:
                raise CacheFull(f"slot {slot}: {int(self.lengths[slot])} cached + {n_new} new "
                                f"tokens exceed the longest sequence allowed ({self.max_len})")
        for g in self._kv_groups:
            need = sum(g.blocks_needed(s, int(self.lengths[s]) + n) for s, n in entries)
            if need > g.pool.free_count:
                raise CacheFull(f"the step needs {need} more cache blocks of {self.block_tokens} "
                                f"tokens, only {g.pool.free_count} of {g.pool.n_blocks} are free")
        for g in self._kv_groups:
            for s, n in entries:
                g.grow(s, int(self.lengths[s]) + n)
            g.flush()

    def end_step(self, entries: Sequence[Tuple[int, int]]) -> None:
        for slot, n_new in entries:
            self.lengths[slot] += n_new
            for g in self._kv_groups:
                g.release_outside_window(slot, int(self.lengths[slot]))
        for g in self._kv_groups:
            g.flush()

    def reserve(self, slot: int, total_len: int, flush: bool = True) -> None:
        """Map blocks for ``total_len`` positions now, so later steps change no table.
        ``flush=False`` leaves the device's copy of the tables for a later call (another
        ``reserve`` or ``begin_step``) to bring up to date: a batch reserves all its slots and
        copies once."""
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not in use")
        if total_len > self.max_len:
            raise CacheFull(f"slot {slot}: {total_len} tokens exceed the longest sequence "
                            f"allowed ({self.max_len})")
        olds = []
        try:
            for g in self._kv_groups:
                if g.request.window > 0:
                    continue
                olds.append((g, int(g.n_blocks_of[slot])))
                g.grow(slot, total_len)
        except CacheFull:
            for g, old in olds:
                g.shrink_to(slot, old)
            raise
        if flush:
            for g in self._kv_groups:
                g.flush()

    # -- views -----------------------------------------------------------------
    def kv_view(self, cache_id: int) -> KVView:
        g, i = self._kv_of[cache_id]
        return KVView(g.k[i], g.v[i], g.table, g.block_tokens, g.request.window)

    def state_view(self, cache_id: int) -> torch.Tensor:
        return self._state[cache_id]

    def has_kv(self, cache_id: int) -> bool:
        return cache_id in self._kv_of

    def has_state(self, cache_id: int) -> bool:
        return cache_id in self._state

    # -- accounting ----------------------------------------------------------------
    def stats(self) -> dict:
        kv_bytes = sum(g.k.numel() * g.k.element_size() * 2 for g in self._kv_groups)
        state_bytes = sum(t.numel() * t.element_size() for t in self._state.values())
        return {
            "block_tokens": self.block_tokens,
            "blocks": self.n_blocks,
            "blocks_free": [g.pool.free_count for g in self._kv_groups],
            "slots": self.max_slots,
            "slots_live": len(self.slots.live()),
            "kv_bytes": kv_bytes,
            "state_bytes": state_bytes,
            "groups": [{"num_kv_heads": g.request.num_kv_heads, "head_dim": g.request.head_dim,
                        "window": g.request.window, "layers": len(g.cache_ids)}
                       for g in self._kv_groups],
        }

    def check(self) -> None:
        """Every block is free or mapped by exactly one live slot; no slot is lost."""
        self.slots.check()
        for g in self._kv_groups:
            g.pool.check()
            mapped: List[int] = []
            for s in range(self.max_slots):
                row = g.table_host[s]
                held = row[row >= 0].tolist()
                if held and not self.slots.is_live(s):
                    raise CacheError(f"free slot {s} still maps blocks {held}")
                mapped.extend(held)
            if len(set(mapped)) != len(mapped):
                raise CacheError("a block is mapped by two sequences")
            if len(mapped) != g.pool.held_count:
                raise CacheError(f"{g.pool.held_count} blocks are held but {len(mapped)} are mapped")
