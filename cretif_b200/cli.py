"""Command line, in the manner of the reference's ``cuinfer`` program
(src/main.cu:14-21, 196-236)::

    python -m cretif_b200 <model_dir> [prompt] [max_tokens] [--dump-logits [file.json]]

``model_dir`` holds config.json and model.safetensors (the reference takes a GGUF
file).  ``prompt`` is text when the folder has a tokenizer.json, else token ids
separated by commas or spaces; default "Once upon a time" (src/main.cu:229-231), or
the model's first token id without a tokenizer.  ``max_tokens`` defaults to 50
(:232-234).  ``--dump-logits`` runs the prompt only and writes the 20 largest logits
of its last position as JSON (:242-301; default file ``cuinfer_logits.json``).

Added options: ``--temperature``, ``--top-k``, ``--seed`` (the reference's
``generate`` arguments, which its program leaves at their defaults), ``--dtype``,
``--cache-tokens``, ``--stop-ids``, and ``--random-weights SEED`` with ``--preset NAME`` or
``--config FILE``, which first writes a model folder with seeded random weights to
``model_dir``.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional


def _parse_prompt(text: str, tokenizer, bos: Optional[int]) -> List[int]:
    if tokenizer is not None:
        return tokenizer.encode(text, add_special=True)
    parts = text.replace(",", " ").split()
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit("the model folder has no tokenizer.json, so the prompt must be token "
                         f"ids separated by commas or spaces; got {text!r}") from None


def _top_logits(row, k: int, tokenizer):
    import torch
    vals, idx = torch.topk(row, min(k, row.numel()))
    out = []
    for rank, (v, i) in enumerate(zip(vals.tolist(), idx.tolist())):
        out.append({"rank": rank, "token_id": i,
                    "token_string": tokenizer.decode([i]) if tokenizer else "",
                    "logit_value": round(v, 6)})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="cretif_b200", description=__doc__.split("\n\n")[0])
    ap.add_argument("model", help="folder with config.json and model.safetensors")
    ap.add_argument("prompt", nargs="?", default=None)
    ap.add_argument("max_tokens", nargs="?", type=int, default=50)
    ap.add_argument("--dump-logits", nargs="?", const="cuinfer_logits.json", default=None,
                    metavar="FILE")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--cache-tokens", type=int, default=None,
                    help="tokens the cache holds (default: the model's longest sequence)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="write a model folder with random weights to MODEL first")
    ap.add_argument("--config", default=None, help="config.json to use with --random-weights")
    ap.add_argument("--preset", default=None,
                    help="named configuration to use with --random-weights (tiny-a, tiny-b, "
                         "smollm2-135m, smollm2-360m, smollm2-1.7b)")
    ap.add_argument("--stop-ids", default=None,
                    help="comma-separated token ids that end generation (default: the model's "
                         "eos_token_id)")
    args = ap.parse_args(argv)

    if args.random_weights is not None:
        from .weights.random_model import write_random_model
        if args.preset:
            from .config.presets import preset
            raw = preset(args.preset)
        elif args.config:
            with open(args.config, "r", encoding="utf-8") as f:
                raw = json.load(f)
        else:
            raise SystemExit("--random-weights needs --preset NAME or --config FILE")
        write_random_model(args.model, raw, args.random_weights)
        print(f"wrote random weights (seed {args.random_weights}) to {args.model}")

    from .engine import Engine
    from .text import load_tokenizer
    tokenizer = load_tokenizer(args.model)
    t0 = time.time()
    from .config import load_config
    _, cfg, spec = load_config(args.model)
    cache_tokens = args.cache_tokens or spec.max_positions
    engine = Engine(args.model, dtype=args.dtype, max_tokens=cache_tokens, device=args.device)
    st = engine.stats()
    print(f"model: {spec.architecture}, {len(spec.layers)} layers, hidden {spec.hidden_size}, "
          f"vocab {spec.vocab_size}; dtype {st['dtype']}")
    print(f"memory: weights {st['weights_bytes'] / 2**20:.1f} MiB, cache "
          f"{st['cache']['kv_bytes'] / 2**20:.1f} MiB ({st['cache']['blocks']} blocks of "
          f"{st['cache']['block_tokens']} tokens); loaded in {time.time() - t0:.1f} s")

    if args.prompt is None:
        if tokenizer is not None:
            prompt_text = "Once upon a time"
        else:
            prompt_text = str(spec.bos_token_id if spec.bos_token_id is not None else 0)
    else:
        prompt_text = args.prompt
    ids = _parse_prompt(prompt_text, tokenizer, spec.bos_token_id)
    if not ids:
        raise SystemExit("the prompt produced no tokens")

    import torch
    if args.dump_logits:
        slot = engine.alloc_slot()
        logits = engine.step([(slot, ids)], "last")[0].float().cpu()
        engine.free_slot(slot)
        doc = {"prompt": prompt_text, "input_token_ids": ids,
               "input_token_strings": [tokenizer.decode([i]) for i in ids] if tokenizer else [],
               "num_input_tokens": len(ids), "logits_position": len(ids) - 1, "top_k": 20,
               "top_logits": _top_logits(logits, 20, tokenizer)}
        with open(args.dump_logits, "w", encoding="utf-8") as f:
            json.dump(doc, f, indent=2)
        print(f"wrote the top 20 logits of position {len(ids) - 1} to {args.dump_logits}")
        return 0

    torch.cuda.synchronize()
    t0 = time.time()
    stops = None if args.stop_ids is None else [int(t) for t in args.stop_ids.split(",") if t]
    res = engine.generate([ids], max_tokens=args.max_tokens, temperature=args.temperature,
                          top_k=args.top_k, seed=args.seed, stop_ids=stops)[0]
    torch.cuda.synchronize()
    dt = time.time() - t0
    print(f"prompt ids: {ids}")
    print(f"generated ids: {res.tokens}  (finish: {res.finish_reason})")
    if tokenizer is not None:
        print(tokenizer.decode(res.tokens))
    total = len(ids) + len(res.tokens) - 1          # as src/main.cu:317-324 counts
    print(f"{total} tokens in {dt * 1e3:.1f} ms: {total / dt:.1f} tok/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
