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


def rel_err(got, want):
    """max |difference| over max |plain logit|."""
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / np.abs(want).max())
