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
against the measured copy bandwidth.  ``points`` holds decode at batch 1 and 64 and, at
the headline batch, at contexts of about 3,072 and 4,096 (``points_roofline_frac``: the same
fraction for each); ``prefill_b8`` and ``prefill_b64`` are steps over 8 and 64 prompts of
2,048 tokens; ``shares`` says where a decode step's time goes (each kind of kernel alone).
``--size 360m --unequal`` decodes after prompts of unequal lengths 256..2,048;
``--dtype float32`` measures the true 32-bit path.
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


def run_decode(engine, batch, steps, warmup, prompt_len, seed=0, unequal=False, shares=False):
    """Prefill `batch` prompts, then time `steps` graph-replayed decode steps.
    Returns (ms_per_step, mean context during the timed steps, launches per step[, shares])."""
    import numpy as np
    import torch
    from cretif_b200.csrc import ops
    from cretif_b200.engine.generate import EngineBackend
    from cretif_b200.sampling import SamplingParams
    rng = np.random.default_rng(seed)
    lengths = [prompt_len] * batch
    if unequal and batch > 1:                 # 256 .. prompt_len, the longest one present
        lengths = [prompt_len] + rng.integers(256, prompt_len + 1, size=batch - 1).tolist()
    prompts = [rng.integers(0, engine.vocab_size, size=n).tolist() for n in lengths]
    be = EngineBackend(engine, SamplingParams(0.0, 0, 42), use_graph=True, run_ahead=False)
    extra = warmup + steps + 1
    be.start_batch(list(range(batch)), prompts, [n + extra for n in lengths])
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
        ctx0 = float(np.mean([cache.lengths[s] for s in be.slots]))
        longest = int(max(cache.lengths[s] for s in be.slots))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            engine.run(slots, lambda: runner.run(longest + i + 1))
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / steps
        engine.check_fault()
        mean_ctx = ctx0 + (steps - 1) / 2.0 + 1
        if shares:
            return ms, mean_ctx, per_step, decode_shares(engine, runner, batch, longest + steps)
        return ms, mean_ctx, per_step
    finally:
        be.end_batch()


def decode_shares(engine, runner, batch, context):
    """Where a decode step's time goes: each kind of kernel of the step alone — every layer's
    launch of that kind, on the model's own weights and cache, captured as one CUDA graph
    and replayed — in microseconds per step.  Alone, a kernel's weight fetch no longer
    overlaps its predecessor's tail, so the parts add up to more than the step."""
    import torch
    from cretif_b200.csrc import ops
    model = engine.model
    b = runner.bufs[batch]
    ctx = engine.context(T=batch, B=batch, tok_ids=b["tok_ids"], tok_pos=b["tok_pos"],
                         tok_seq=b["tok_seq"], seq_slot=b["seq_slot"], seq_start=b["seq_start"],
                         cu_seqlens=b["cu"], is_decode=True, max_new=1, max_context=context)
    layers = []
    for i, entry in enumerate(model.spec.schedule):
        layer = model.layers[entry.layer]
        caches = model.layer_caches(i, engine.cache)
        mix = next(k for k, br in enumerate(layer.branches) if br.role == "mixer")
        ffn = next(k for k, br in enumerate(layer.branches) if br.role == "feed_forward")
        layers.append((layer.branches[mix], caches[mix], layer.branches[ffn]))
    a0 = layers[0][0].part
    dev = engine.device
    h = torch.zeros((batch, model.spec.hidden_size), dtype=torch.float32, device=dev)
    ops.embed_rows(model.embedding.table, b["tok_ids"], h, engine.fault)
    q = torch.zeros((batch, a0.q_dim), dtype=engine.dtype, device=dev)
    o = torch.zeros((batch, a0.q_dim), dtype=engine.dtype, device=dev)
    act = torch.zeros((batch, layers[0][2].part.inter), dtype=engine.dtype, device=dev)
    logits = torch.zeros((batch, engine.vocab_size), dtype=torch.float32, device=dev)
    sampled = torch.zeros(batch, dtype=torch.int32, device=dev)

    def qkv(mb, cache, fb):
        a, (w, eps), kv = mb.part, mb.norm.rms_params(), cache.kv
        cos, sin, pairing, _ = a.position.rotary_table()
        ops.fused_qkv_rope(h, w, eps, a.w_qkv, q, cos, sin, pairing, a.nh, a.nkv, a.hd,
                           ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.table, kv.k, kv.v,
                           kv.block_tokens, True, ctx.fault)

    def attention(mb, cache, fb):
        mb.part.attend(q, o, ctx, cache.kv)

    def o_proj(mb, cache, fb):
        ops.fused_linear_add(o, mb.part.w_o, h)

    def gate_up(mb, cache, fb):
        f, (w, eps) = fb.part, fb.norm.rms_params()
        ops.fused_gate_up_silu(h, w, eps, f.w_gate_up, act, f.gu_block)

    def down(mb, cache, fb):
        ops.fused_linear_add(act, fb.part.w_down, h)

    def head_and_sample():
        w, eps = model.final_norm.rms_params()
        ops.fused_norm_linear(h, w, eps, model.head.weight, logits)
        runner.sampler(logits, sampled, b["request"], b["draw"])

    def timed(fn):
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
        torch.cuda.synchronize()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            g.replay()
        a.record()
        for _ in range(10):
            g.replay()
        z.record()
        torch.cuda.synchronize()
        h.zero_()                 # the residual additions of the replays may have overflowed
        return a.elapsed_time(z) * 100.0          # microseconds per replay
    out = {}
    try:
        for name, fn in (("qkv", qkv), ("attention", attention), ("o_proj", o_proj),
                         ("gate_up", gate_up), ("down", down)):
            out[name] = timed(lambda fn=fn: [fn(*t) for t in layers])
        out["head_and_sample"] = timed(head_and_sample)
    except Exception as e:        # a model whose parts are not the fused bfloat16 ones
        return {"unavailable": " ".join(str(e).split())[:200]}
    out["unit"] = "us per step, each kind of kernel alone"
    return out


def run_prefill(engine, tokens, repeats, warmup, batch=1):
    """One step over `batch` prompts of `tokens` ids through Engine.step, timed with CUDA
    events.  (A step shape that repeats is replayed as a CUDA graph from its third call on;
    the host-to-device copy of the token ids is inside the timed region.)"""
    import numpy as np
    import torch
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, engine.vocab_size, size=tokens).tolist() for _ in range(batch)]
    times = []
    for i in range(warmup + repeats):
        slots = [engine.alloc_slot() for _ in range(batch)]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step(list(zip(slots, prompts)), "last", check=False)
        b.record()
        torch.cuda.synchronize()
        for s in slots:
            engine.free_slot(s)
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
    ap.add_argument("--skip-points", action="store_true",
                    help="only the headline decode, the 2,048-token prefill and e2e")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="measure one phase only and print a short line (a small workload, "
                         "for instance under a profiler)")
    ap.add_argument("--size", default="135m", choices=sorted(SIZES),
                    help="layer sizes: SmolLM2-135M (the headline), 360M or 1.7B")
    ap.add_argument("--no-shares", action="store_true",
                    help="skip the per-kernel shares of the decode step")
    ap.add_argument("--unequal", action="store_true",
                    help="prompts of unequal lengths 256..2,048 instead of 2,048 each")
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
    points_on = not args.skip_points and args.only is None

    tmp = tempfile.mkdtemp(prefix="cretif_bench_")
    try:
        write_random_model(tmp, cfg, seed=1234)
        max_batch = max(args.batch, 64) if points_on else args.batch
        engine = Engine(tmp, dtype=args.dtype, max_tokens=max_batch * CONTEXT + 64 * 64,
                        max_len=CONTEXT)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    def step_bytes(batch, mean_ctx):
        """What a decode step has to read: every weight once, the live requests' cache."""
        return (nums["matmul_params"] * wbytes + nums["norm_params"] * 4
                + batch * mean_ctx * nums["kv_bytes_per_token"] * (wbytes // 2))

    def hbm_frac(batch, mean_ctx, ms):
        return step_bytes(batch, mean_ctx) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]

    T = PROMPT_LEN
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]

    def prefill_record(batch, repeats=5, warmup=3):
        ms = run_prefill(engine, T, repeats=repeats, warmup=warmup, batch=batch)
        flops = batch * (2 * T * (nums["matmul_params"] - cfg["vocab_size"] * cfg["hidden_size"])
                         + 2 * cfg["vocab_size"] * cfg["hidden_size"]      # the head: last rows
                         + layers * nh * 2 * hd * T * (T + 1))             # causal QK^T and PV
        return {"value": batch * T / (ms * 1e-3), "tokens": batch * T, "ms": ms,
                "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "flops": flops}

    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "batch": args.batch,
                          **prefill_record(args.batch, repeats=max(1, min(args.steps, 5)),
                                           warmup=max(1, min(args.warmup, 3)))}))
        return 0

    with ClockSampler() as clocks:
        out = run_decode(engine, args.batch, steps, args.warmup, PROMPT_LEN,
                         unequal=args.unequal, shares=not args.no_shares)
    ms, mean_ctx, per_step = out[:3]
    shares = out[3] if len(out) > 3 else None
    value = args.batch / (ms * 1e-3)
    if args.only == "decode":
        print(json.dumps({"only": "decode", "batch": args.batch, "value": value,
                          "ms_per_step": ms, "frac": hbm_frac(args.batch, mean_ctx, ms),
                          "shares": shares}))
        return 0

    rest = ClockSampler()
    rest.__enter__()           # the clocks under everything below, which runs much hotter
    prefill = prefill_record(1)
    points, fracs, more = {}, {}, {}
    if points_on:
        few = min(256, steps)
        for b, name in ((1, "decode_b1"), (64, "decode_b64")):
            pms, pctx, _ = run_decode(engine, b, few, args.warmup, PROMPT_LEN, seed=b,
                                      unequal=args.unequal)
            points[name] = b / (pms * 1e-3)
            fracs[name] = hbm_frac(b, pctx, pms)
        # decoding at longer contexts (the batch of the headline), and whole batches of prompts
        for ctx_at in (3072, 4096):
            n = min(64, steps)
            pms, pctx, _ = run_decode(engine, args.batch, n, args.warmup,
                                      ctx_at - args.warmup - n - 1, seed=ctx_at)
            points[f"decode_b{args.batch}_ctx{ctx_at}"] = args.batch / (pms * 1e-3)
            fracs[f"decode_b{args.batch}_ctx{ctx_at}"] = hbm_frac(args.batch, pctx, pms)
        for b in (8, 64):
            more[f"prefill_b{b}"] = prefill_record(b, repeats=3, warmup=2)

    e2e = run_e2e(engine, args.batch, min(steps, 512), PROMPT_LEN)
    rest.__exit__(None, None, None)

    achieved = step_bytes(args.batch, mean_ctx) / (ms * 1e-3) / 1e9
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
                   "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch,
                   "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "mean_context_timed": mean_ctx,
                   "prompts": "unequal 256..2048" if args.unequal else "equal",
                   "parallelism": "none", "weights": "random N(0,0.02), seed 1234",
                   "cache_block_tokens": 64,
                   "l2": "weights+cache read per step exceed L2, no flush",
                   "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "bytes": step_bytes(args.batch, mean_ctx), "of": pk["source"]},
        "points": points,
        "points_roofline_frac": fracs,
        "shares": shares,
        **more,
        "e2e": e2e,
        "gpu_launches": per_step * steps,
        "launches_per_step": per_step,
        "clocks": clocks.result,
        "clocks_other_points": rest.result,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
