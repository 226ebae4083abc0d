#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
    python bench.py --impl reference ...      # the reference arm (see reference_arm)

The model has the layer sizes of SmolLM2-135M (30 layers, width 576, 9 heads on 3
key/value heads of 64, feed-forward 1536, vocabulary 49152, tied head) with seeded
random weights; prompts are 2,048 uniform token ids per sequence and decoding runs on
from there, so the context grows from 2,048 towards 4,096.  A "step" is one decode
step of the whole batch, replayed as a CUDA graph and timed with CUDA events on the
launching stream.  ``value`` is decoded tokens per second at the default batch of 8;
``e2e`` is the same through ``Engine.generate`` with host token lists in and out;
``prefill`` is one step over a 2,048-token prompt; ``roofline`` is the bytes a decode
step has to read (every weight once plus the live requests' cache) over its time,
against the measured copy bandwidth; ``points`` holds decode at batch 1 and 64.
Every weight plus the cache exceed the L2 cache, so no flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from cretif_b200.config.presets import preset as _preset  # noqa: E402

SMOLLM2_135M = _preset("smollm2-135m")
SIZES = {"135m": "smollm2-135m", "360m": "smollm2-360m", "1.7b": "smollm2-1.7b"}
PROMPT_LEN = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        self.proc = None
        exe = shutil.which("nvidia-smi")
        if exe:
            self.proc = subprocess.Popen(
                [exe, "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            cols = [c.strip() for c in line.split(",")]
            if len(cols) < 6:
                continue
            try:
                sm.append(float(cols[0])); mx.append(float(cols[1]))
            except ValueError:
                continue
            for n, c in zip(names, cols[2:6]):
                if c.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx),
                           "reasons": sorted(reasons)}


def model_numbers(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh * hd + 2 * nkv * hd) * H + H * nh * hd + 3 * I * H
    matmul_params = layers * per_layer + V * H
    return {"matmul_params": matmul_params, "norm_params": (2 * layers + 1) * H,
            "kv_bytes_per_token": layers * 2 * nkv * hd * 2, "per_layer": per_layer}


def run_decode(engine, batch, steps, warmup, prompt_len, seed=0):
    """Prefill `batch` prompts, then time `steps` graph-replayed decode steps.
    Returns (ms_per_step, mean context during the timed steps, launches per step)."""
    import numpy as np
    import torch
    from cretif_b200.csrc import ops
    from cretif_b200.engine.generate import EngineBackend
    from cretif_b200.sampling import SamplingParams
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, engine.vocab_size, size=prompt_len).tolist() for _ in range(batch)]
    be = EngineBackend(engine, SamplingParams(0.0, 0, 42), use_graph=True, run_ahead=False)
    total = prompt_len + warmup + steps + 1
    be.start_batch(list(range(batch)), prompts, [total] * batch)
    try:
        be.prefill()
        active = list(range(batch))
        before = ops.launch_count()
        be.decode(active)                       # captures the graph
        per_step = (ops.launch_count() - before) // 2    # warm-up pass + captured pass
        for _ in range(max(0, warmup - 1)):
            be.decode(active)
        cache, runner = engine.cache, be.runner
        slots = [(s, 1) for s in be.slots]
        torch.cuda.synchronize()
        ctx0 = int(cache.lengths[be.slots[0]])
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            cache.begin_step(slots)
            runner.run()
            cache.end_step(slots)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / steps
        engine.check_fault()
        return ms, ctx0 + (steps - 1) / 2.0 + 1, per_step
    finally:
        be.end_batch()


def run_prefill(engine, tokens, repeats, warmup):
    """One step over a prompt of `tokens` ids through Engine.step, timed with CUDA events.
    (A step shape that repeats is replayed as a CUDA graph from its third call on; the
    host-to-device copy of the token ids is inside the timed region.)"""
    import numpy as np
    import torch
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, engine.vocab_size, size=tokens).tolist()
    times = []
    for i in range(warmup + repeats):
        slot = engine.alloc_slot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([(slot, prompt)], "last", check=False)
        b.record()
        torch.cuda.synchronize()
        engine.free_slot(slot)
        if i >= warmup:
            times.append(a.elapsed_time(b))
    engine.check_fault()
    return statistics.median(times)


def run_e2e(engine, batch, steps, prompt_len):
    import numpy as np
    import torch
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, engine.vocab_size, size=prompt_len).tolist() for _ in range(batch)]
    for _ in range(2):      # warm-up: the decode graph, and the prefill step's on its second run
        engine.generate(prompts, max_tokens=4, stop_ids=[])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = engine.generate(prompts, max_tokens=steps, stop_ids=[])
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n = sum(len(r.tokens) for r in res)
    # the same call cut after the first token: what of `seconds` is the prompts' prefill
    t0 = time.perf_counter()
    first = engine.generate(prompts, max_tokens=1, stop_ids=[])
    torch.cuda.synchronize()
    dt1 = time.perf_counter() - t0
    n1 = sum(len(r.tokens) for r in first)
    h2d = batch * prompt_len * 4 + 8 * batch * 4          # prompts once + the decode batch state
    out = {"value": n / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d / steps,
           "d2h_bytes_per_step": batch * 4, "seconds": dt, "tokens": n,
           "includes": "prefill of the prompts, every decode step's device-to-host read of "
                       "the sampled ids",
           "prefill_seconds": dt1}
    if n > n1 and dt > dt1:
        out["decode_only"] = (n - n1) / (dt - dt1)       # tokens/s after the first token
    return out


def probe(engine, args) -> int:
    """A small eager workload for profilers: `--probe decode` runs --steps decode steps of
    --batch sequences without a CUDA graph after a 2,048-token prefill; `--probe prefill`
    runs --steps prefills of one 2,048-token prompt."""
    import numpy as np
    import torch
    from cretif_b200.engine.generate import EngineBackend
    from cretif_b200.sampling import SamplingParams
    if args.probe == "prefill":
        ms = run_prefill(engine, PROMPT_LEN, repeats=max(1, args.steps), warmup=1)
        print(f"prefill of {PROMPT_LEN} tokens: {ms:.3f} ms")
        return 0
    rng = np.random.default_rng(0)
    B = args.batch
    prompts = [rng.integers(0, engine.vocab_size, size=PROMPT_LEN).tolist() for _ in range(B)]
    be = EngineBackend(engine, SamplingParams(), use_graph=False)
    be.start_batch(list(range(B)), prompts, [PROMPT_LEN + args.steps + 8] * B)
    try:
        be.prefill()
        active = list(range(B))
        be.decode(active)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            be.decode(active)
        torch.cuda.synchronize()
        print(f"eager decode, batch {B}: {(time.perf_counter() - t0) * 1e3 / args.steps:.3f} "
              "ms/step (launch-bound without the graph)")
    finally:
        be.end_batch()
    return 0


def reference_arm(args) -> int:
    """The unmodified reference (CuInfer), built from its own sources by
    ``baseline/reference_tools.py`` into ``baseline/_ref/cuinfer``, run through its stock command
    line ``cuinfer <gguf> <prompt> <n>``.  It serves one sequence at a time, in float32, with
    a context of at most 2,048 positions, so its arm is batch 1 with a 1,024-token prompt: the
    closest it can do.  Two runs that differ only in the number of new tokens give the decode
    rate (its own timer covers prefill + decoding; the difference leaves the decoding)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_tools as ref
    why = ref.available()
    if why is None and args.gpus != 1:
        why = "the reference runs on one GPU only"
    if why is None:
        import torch
        if not torch.cuda.is_available():
            why = "no CUDA device here (the reference binary is built and needs a GPU)"
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    import numpy as np
    from cretif_b200.weights.random_model import write_random_model
    cfg = _preset(SIZES[args.size])
    cfg["rope_interleaved"] = True
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    prompt_len, first = 1024, max(args.warmup, 3)
    steps = max(args.steps, 128)
    steps = min(steps, 2048 - prompt_len - first - 1)
    tmp = tempfile.mkdtemp(prefix="cretif_ref_")
    try:
        write_random_model(tmp, cfg, seed=1234)
        gguf = os.path.join(tmp, "model.gguf")
        ref.write_gguf(tmp, gguf)
        chars = ref.char_ids(cfg["vocab_size"])
        rng = np.random.default_rng(0)
        ids = [chars[i] for i in rng.integers(0, len(chars), size=prompt_len)]
        prompt = ref.prompt_for(ids, cfg["vocab_size"])
        with ClockSampler() as clocks:
            short = ref.generate(gguf, prompt, first)
            long_ = ref.generate(gguf, prompt, first + steps)
    except Exception as e:          # a build that does not run here, a fault of the reference
        print(json.dumps({"impl": "reference",
                          "unavailable": "the reference did not run: "
                                         + " ".join(str(e).split())[:300]}))
        return 0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    new = long_["positions"] - short["positions"]
    ms = long_["ms"] - short["ms"]
    if new <= 0 or ms <= 0:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference stopped early (its end-of-sequence id was sampled)"}))
        return 0
    line = {
        "metric": f"decode tokens/s (SmolLM2-{args.size.upper()} sizes, random weights, batch 1)",
        "value": new / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": new,
        "warmup": first, "ms_per_step": ms / new, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "reference",
        "same_config": False,
        "config": {"model": f"SmolLM2-{args.size.upper()} sizes (Llama)",
                   "layers": cfg["num_hidden_layers"], "global_batch": 1,
                   "prompt_len": prompt_len, "seq_len": prompt_len + first + steps,
                   "weights": "random N(0,0.02), seed 1234, as F32 GGUF",
                   "why_not_the_same": "the reference serves one sequence, in float32, up to "
                                       "2,048 positions",
                   "timing": "the reference's own timer; difference of two runs"},
        "e2e": {"value": long_["positions"] / (long_["ms"] * 1e-3), "unit": "positions/s",
                "includes": "prefill of 1,024 tokens and decoding, text in and text out"},
        "clocks": clocks.result,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--size", default="135m", choices=sorted(SIZES),
                    help="layer sizes: SmolLM2-135M (the headline), 360M or 1.7B")
    ap.add_argument("--probe", choices=["decode", "prefill"], default=None,
                    help="run a few eager steps of one phase and print their time (for "
                         "profilers); no JSON line")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported (the engine is "
              "single-GPU by design)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from cretif_b200.csrc import ops
    from cretif_b200.engine import Engine
    from cretif_b200.weights.random_model import write_random_model

    cfg = _preset(SIZES[args.size])
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    steps = min(args.steps, CONTEXT - PROMPT_LEN - args.warmup - 1)
    pk = peaks()
    nums = model_numbers(cfg, layers)
    wbytes = 2 if args.dtype == "bfloat16" else 4

    tmp = tempfile.mkdtemp(prefix="cretif_bench_")
    try:
        write_random_model(tmp, cfg, seed=1234)
        max_batch = args.batch if args.skip_points else max(args.batch, 64)
        engine = Engine(tmp, dtype=args.dtype, max_tokens=max_batch * CONTEXT + 64 * 64,
                        max_len=CONTEXT)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    if args.probe:
        return probe(engine, args)

    with ClockSampler() as clocks:
        ms, mean_ctx, per_step = run_decode(engine, args.batch, steps, args.warmup, PROMPT_LEN)
    value = args.batch / (ms * 1e-3)
    step_bytes = (nums["matmul_params"] * wbytes + nums["norm_params"] * 4
                  + args.batch * mean_ctx * nums["kv_bytes_per_token"] * (wbytes // 2))
    achieved = step_bytes / (ms * 1e-3) / 1e9

    pre_ms = run_prefill(engine, PROMPT_LEN, repeats=5, warmup=3)
    T = PROMPT_LEN
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
    flops = 2 * T * (nums["matmul_params"] - cfg["vocab_size"] * cfg["hidden_size"]) \
        + 2 * cfg["vocab_size"] * cfg["hidden_size"] \
        + layers * nh * 2 * hd * T * (T + 1)          # causal QK^T and PV
    prefill = {"value": T / (pre_ms * 1e-3), "tokens": T, "ms": pre_ms,
               "frac": flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "flops": flops}

    points = {}
    if not args.skip_points:
        for b, name in ((1, "decode_b1"), (64, "decode_b64")):
            pms, _, _ = run_decode(engine, b, min(256, steps), args.warmup, PROMPT_LEN, seed=b)
            points[name] = b / (pms * 1e-3)

    e2e = run_e2e(engine, args.batch, min(steps, 512), PROMPT_LEN)

    line = {
        "metric": f"decode tokens/s (SmolLM2-{args.size.upper()} sizes, random weights, batch "
                  f"{args.batch}, context 2048->4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"SmolLM2-{args.size.upper()} sizes (Llama)", "layers": layers,
                   "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
                   "heads": nh, "kv_heads": cfg["num_key_value_heads"], "head_dim": hd,
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch, "prompt_len": PROMPT_LEN,
                   "seq_len": CONTEXT, "mean_context_timed": mean_ctx, "parallelism": "none",
                   "weights": "random N(0,0.02), seed 1234", "cache_block_tokens": 64,
                   "l2": "weights+cache read per step exceed L2, no flush",
                   "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "bytes": step_bytes,
                     "of": pk["source"]},
        "points": points,
        "e2e": e2e,
        "gpu_launches": per_step * steps,
        "launches_per_step": per_step,
        "clocks": clocks.result,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
