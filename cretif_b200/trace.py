"""Trace replay: feed given token ids through the engine step by step, write logits.

Nothing is sampled.  The replay drives the same :class:`~cretif_b200.engine.Engine`
that generation uses: its model, step function, cache and kernels.  It plays the part
of the reference's ``--dump-logits`` mode (src/main.cu:242-301), which runs one
prefill and writes the top logits of the last position; here every step of a request
can be replayed and whole rows of logits are written.

Input: one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives each request's next tokens and the places among them whose logits
are wanted; the requests of a step either all start or all go on by one token.
``end`` lists requests that are finished after the step; their cache is given back.
For a step that wants something, ``<out>/<step>.f32`` holds the logits
``[wanted, vocab]`` as little-endian float32, in the order of the entries and of
``want``.  After every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict



def replay(engine, lines, out_dir: str, report=print) -> int:
    """Run the steps read from ``lines``; returns the number of steps run."""
    os.makedirs(out_dir, exist_ok=True)
    slot_of: Dict[str, int] = {}
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step = msg["step"]
        entries, want = [], []
        for e in msg.get("entries", []):
            rid = str(e["id"])
            if rid not in slot_of:
                slot_of[rid] = engine.alloc_slot()
            entries.append((slot_of[rid], e["tokens"]))
            want.append(list(e.get("want", [])))
        if entries:
            logits = engine.step(entries, want)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for rid in msg.get("end", []):
            rid = str(rid)
            if rid in slot_of:
                engine.free_slot(slot_of.pop(rid))
        report(f"done {step}")
        n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(
        prog="trace_run", description="Replay token ids through the engine and write logits.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from .engine import Engine
    engine = Engine(args.model, dtype=args.dtype, max_tokens=args.max_tokens, device=args.device)

    def report(text):
        sys.stdout.write(text + "\n")
        sys.stdout.flush()
    replay(engine, sys.stdin, args.out, report)
    return 0
