"""The ways of cutting the same requests into steps that the GPU tests compare."""
import numpy as np
import torch


def run_whole(engine, toks):
    """One request alone, all tokens in one step, logits at every place."""
    slot = engine.alloc_slot()
    try:
        return engine.step([(slot, toks)], "all").cpu().numpy()
    finally:
        engine.free_slot(slot)


def run_tail_by_one(engine, toks, tail=32):
    """One request alone: all but the last ``tail`` tokens in one step, then one by one."""
    slot = engine.alloc_slot()
    try:
        n = len(toks)
        first = max(1, n - tail)
        rows = [engine.step([(slot, toks[:first])], "all").cpu().numpy()]
        for i in range(first, n):
            rows.append(engine.step([(slot, [toks[i]])], "all").cpu().numpy())
        return np.concatenate(rows, axis=0)
    finally:
        engine.free_slot(slot)


def run_batch(engine, requests, prompt_lens):
    """Requests that start together: request r brings its first prompt_lens[r] tokens in
    step 0, then one token a step until its tokens run out; shorter ones leave earlier.
    Returns the logits of every place of every request."""
    slots = [engine.alloc_slot() for _ in requests]
    out = [np.zeros((len(t), engine.vocab_size), dtype=np.float32) for t in requests]
    try:
        entries = [(slots[r], requests[r][:prompt_lens[r]]) for r in range(len(requests))]
        logits = engine.step(entries, "all").cpu().numpy()
        o = 0
        for r, p in enumerate(prompt_lens):
            out[r][:p] = logits[o:o + p]
            o += p
        fed = list(prompt_lens)
        live = [r for r in range(len(requests)) if fed[r] < len(requests[r])]
        for r in range(len(requests)):
            if r not in live:
                engine.free_slot(slots[r]); slots[r] = None
        while live:
            entries = [(slots[r], [requests[r][fed[r]]]) for r in live]
            logits = engine.step(entries, "all").cpu().numpy()
            for i, r in enumerate(live):
                out[r][fed[r]] = logits[i]
                fed[r] += 1
            for r in list(live):
                if fed[r] >= len(requests[r]):
                    live.remove(r)
                    engine.free_slot(slots[r]); slots[r] = None
        return out
    finally:
        for s in slots:
            if s is not None:
                engine.free_slot(s)


def run_chunks(engine, toks, chunks):
    """One request alone, fed as chunks of the given sizes (the rest as a last chunk)."""
    slot = engine.alloc_slot()
    try:
        rows, at = [], 0
        sizes = list(chunks)
        while at < len(toks):
            n = sizes.pop(0) if sizes else len(toks) - at
            n = min(n, len(toks) - at)
            rows.append(engine.step([(slot, toks[at:at + n])], "all").cpu().numpy())
            at += n
        return np.concatenate(rows, axis=0)
    finally:
        engine.free_slot(slot)


def run_schedule(engine, requests, schedule):
    """Any mixture: ``schedule`` is a list of steps, each a list of (request index, number of
    tokens); a request starts at its first appearance, is fed in the chunks given and its
    slot is given back when its tokens are used up.  Returns the logits of every place."""
    slots = {}
    fed = [0] * len(requests)
    out = [np.zeros((len(t), engine.vocab_size), dtype=np.float32) for t in requests]
    try:
        for step in schedule:
            entries = []
            for r, n in step:
                if r not in slots:
                    slots[r] = engine.alloc_slot()
                entries.append((slots[r], requests[r][fed[r]:fed[r] + n]))
            logits = engine.step(entries, "all").cpu().numpy()
            o = 0
            for r, n in step:
                out[r][fed[r]:fed[r] + n] = logits[o:o + n]
                o += n
                fed[r] += n
                if fed[r] >= len(requests[r]):
                    engine.free_slot(slots.pop(r))
        assert all(f == len(t) for f, t in zip(fed, requests)), "the schedule leaves tokens unfed"
        return out
    finally:
        for s in slots.values():
            engine.free_slot(s)


def rel_err(got, want):
    """max |difference| over max |plain logit|."""
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / np.abs(want).max())
