"""Running the unmodified reference engine (CuInfer) beside this library.

The reference is a CMake C++/CUDA program that reads GGUF files and takes a text prompt.
Nothing of it is part of the product; these helpers exist for two jobs only:

* ``tests/golden/make_reference_golden.py`` runs its stock ``cuinfer <gguf> <prompt>
  --dump-logits`` on tiny random models and commits the logits it prints, so that the plain
  implementation under ``tests/`` is pinned by the reference's own output;
* ``bench.py --impl reference`` times its stock ``cuinfer <gguf> <prompt> <n>``.

What is needed for that, and nothing more:

* :func:`build_reference` compiles the reference's sources as they are with ``nvcc`` for
  sm_100a (its CMake project fetches googletest from the network for its tests; the program
  itself needs none of it) into ``baseline/_ref/cuinfer``;
* :func:`write_gguf` writes a model folder of this library (config.json + safetensors) as an
  F32 GGUF file with the metadata keys the reference reads (src/model.cu:536-548,
  src/gguf_parser.cpp:694-765; container layout src/gguf_parser.cpp:530-615) and a byte-level
  vocabulary without merges, under which a prompt of printable ASCII characters encodes to
  one known token id per character (src/tokenizer.cpp:341-424, 437-466);
* :func:`prompt_for` / :func:`char_ids` translate between such prompts and token ids.

The reference rotates pairs ``(2j, 2j+1)`` of the rows as stored (src/kernels/
elementwise.cu:232-258), so a model folder run through it corresponds to this library's
``rope_interleaved: true``.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import struct
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
BINARY = os.path.join(REF_DIR, "cuinfer")
CHARS = [chr(c) for c in range(33, 127)]          # '!' .. '~': bytes that map to themselves

# GGUF value types (src/gguf_parser.cpp, enum GGUFValueType)
_U32, _F32, _BOOL, _STR, _ARR = 4, 6, 7, 8, 9


def build_reference(source_dir: str, verbose: bool = True) -> str:
    """Copy ``source_dir``'s ``src/`` and ``include/`` to ``baseline/_ref`` and compile the
    program with nvcc for sm_100a.  Returns the binary's path."""
    for sub in ("src", "include"):
        dst = os.path.join(REF_DIR, sub)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(os.path.join(source_dir, sub), dst)
    sources = []
    for root, _, files in os.walk(os.path.join(REF_DIR, "src")):
        sources += [os.path.join(root, f) for f in sorted(files) if f.endswith((".cu", ".cpp"))]
    cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(REF_DIR, "include"), "-o", BINARY, *sources]
    if verbose:
        print("building the reference:", " ".join(cmd), file=sys.stderr, flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on the reference sources:\n{r.stdout}\n{r.stderr}")
    return BINARY


def available() -> Optional[str]:
    """None if the reference binary can run here, else why not (one line)."""
    if not os.path.isfile(BINARY) or not os.access(BINARY, os.X_OK):
        return (f"the reference binary {os.path.relpath(BINARY, os.path.dirname(HERE))} has "
                "not been built (python baseline/reference_tools.py build <reference dir>)")
    return None


def char_ids(vocab_size: int) -> List[int]:
    """Token id of each of the 94 prompt characters: spread over the vocabulary, fixed."""
    rng = np.random.default_rng(94)
    return sorted(rng.choice(vocab_size, size=len(CHARS), replace=False).tolist())


def prompt_for(ids: Sequence[int], vocab_size: int) -> str:
    """The text that the reference's tokenizer encodes to ``ids`` under :func:`write_gguf`'s
    vocabulary (every id must be one of :func:`char_ids`)."""
    where = {t: c for t, c in zip(char_ids(vocab_size), CHARS)}
    return "".join(where[int(t)] for t in ids)


def _s(text: str) -> bytes:
    raw = text.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


def _kv(key: str, vtype: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", vtype) + payload


def write_gguf(model_dir: str, path: str, context_length: int = 2048) -> Dict[str, int]:
    """Write ``model_dir`` (a Llama model folder of this library) as an F32 GGUF file."""
    from safetensors import safe_open
    import torch
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    V = cfg["vocab_size"]
    if cfg.get("head_dim") not in (None, H // nh):
        raise ValueError("the reference fixes head_dim = hidden_size / heads (src/model.cu:541)")
    tokens = [f"<t{i}>" for i in range(V)]
    for t, c in zip(char_ids(V), CHARS):
        tokens[t] = c
    arch = "llama"
    kvs = [
        _kv("general.architecture", _STR, _s(arch)),
        _kv(f"{arch}.context_length", _U32, struct.pack("<I", context_length)),
        _kv(f"{arch}.embedding_length", _U32, struct.pack("<I", H)),
        _kv(f"{arch}.block_count", _U32, struct.pack("<I", L)),
        _kv(f"{arch}.attention.head_count", _U32, struct.pack("<I", nh)),
        _kv(f"{arch}.attention.head_count_kv", _U32, struct.pack("<I", nkv)),
        _kv(f"{arch}.feed_forward_length", _U32, struct.pack("<I", cfg["intermediate_size"])),
        _kv(f"{arch}.vocab_size", _U32, struct.pack("<I", V)),
        _kv(f"{arch}.rope.freq_base", _F32, struct.pack("<f", cfg.get("rope_theta", 10000.0))),
        _kv(f"{arch}.attention.layer_norm_rms_epsilon", _F32,
            struct.pack("<f", cfg.get("rms_norm_eps", 1e-5))),
        _kv("tokenizer.ggml.model", _STR, _s("gpt2")),
        _kv("tokenizer.ggml.tokens", _ARR,
            struct.pack("<IQ", _STR, V) + b"".join(_s(t) for t in tokens)),
        _kv("tokenizer.ggml.merges", _ARR, struct.pack("<IQ", _STR, 0)),
        _kv("tokenizer.ggml.add_bos_token", _BOOL, struct.pack("<B", 0)),
        _kv("tokenizer.ggml.bos_token_id", _U32, struct.pack("<I", 0)),
        # generation stops at this id (src/model.cu:1082): one no prompt character has
        _kv("tokenizer.ggml.eos_token_id", _U32,
            struct.pack("<I", next(i for i in range(V - 1, -1, -1) if len(tokens[i]) > 1))),
    ]
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight":
             "output_norm.weight", "lm_head.weight": "output.weight"}
    per_layer = {"input_layernorm.weight": "attn_norm.weight",
                 "post_attention_layernorm.weight": "ffn_norm.weight",
                 "self_attn.q_proj.weight": "attn_q.weight",
                 "self_attn.k_proj.weight": "attn_k.weight",
                 "self_attn.v_proj.weight": "attn_v.weight",
                 "self_attn.o_proj.weight": "attn_output.weight",
                 "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
                 "mlp.down_proj.weight": "ffn_down.weight"}
    for i in range(L):
        for ours, theirs in per_layer.items():
            names[f"model.layers.{i}.{ours}"] = f"blk.{i}.{theirs}"
    tensors = []
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for ours in f.keys():
            if ours == "lm_head.weight" and cfg.get("tie_word_embeddings"):
                continue
            arr = f.get_tensor(ours).to(torch.float32).contiguous().numpy()
            tensors.append((names[ours], arr))
    infos, offset = [], 0
    for name, arr in tensors:
        dims = list(reversed(arr.shape))             # ggml order: innermost first
        infos.append(_s(name) + struct.pack("<I", len(dims))
                     + b"".join(struct.pack("<Q", d) for d in dims)
                     + struct.pack("<IQ", 0, offset))     # type 0 = F32
        offset += (arr.nbytes + 31) // 32 * 32
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kvs)) + b"".join(kvs) \
        + b"".join(infos)
    with open(path, "wb") as out:
        out.write(head)
        out.write(b"\0" * (-len(head) % 32))
        for _, arr in tensors:
            out.write(arr.tobytes())
            out.write(b"\0" * (-arr.nbytes % 32))
    return {"tensors": len(tensors), "bytes": os.path.getsize(path)}


def dump_logits(gguf: str, prompt: str, out_json: str, timeout: int = 600) -> dict:
    """The stock ``cuinfer <gguf> <prompt> --dump-logits <file.json>`` (src/main.cu:242-301)."""
    r = subprocess.run([BINARY, gguf, prompt, "--dump-logits", out_json], capture_output=True,
                       text=True, timeout=timeout)
    if r.returncode != 0:
        raise RuntimeError(f"the reference failed ({r.returncode}):\n{r.stdout[-2000:]}\n"
                           f"{r.stderr[-2000:]}")
    with open(out_json) as f:
        return json.load(f)


def generate(gguf: str, prompt: str, max_tokens: int, timeout: int = 1800) -> dict:
    """The stock ``cuinfer <gguf> <prompt> <n>`` (src/main.cu:303-326): its own timing line
    ``Generated <prompt + new> tokens in <ms> ms`` covers prefill and decoding."""
    r = subprocess.run([BINARY, gguf, prompt, str(max_tokens)], capture_output=True, text=True,
                       timeout=timeout)
    if r.returncode != 0:
        raise RuntimeError(f"the reference failed ({r.returncode}):\n{r.stdout[-2000:]}\n"
                           f"{r.stderr[-2000:]}")
    m = re.search(r"Generated (\d+) tokens in ([0-9.]+) ms", r.stdout)
    if not m:
        raise RuntimeError("the reference printed no timing line:\n" + r.stdout[-2000:])
    return {"positions": int(m.group(1)), "ms": float(m.group(2))}


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "build":
        print(build_reference(sys.argv[2]))
    else:
        print("usage: python baseline/reference_tools.py build <directory of the reference>")
        sys.exit(2)
