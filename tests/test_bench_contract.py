"""bench.py's paths that need no GPU: more than one GPU is refused with exit code 2 and one
line; the reference arm prints its one-line JSON record and exits 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args],
                          capture_output=True, text=True, timeout=120, cwd=ROOT)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = _bench("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = _bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and rec["unavailable"]
    assert "\n" not in rec["unavailable"]


def test_gguf_export_for_the_reference(tmp_path):
    """The F32 GGUF file the reference arm and the golden files are made from: header,
    metadata keys, tensor table (dimensions innermost first, 32-byte aligned offsets) and
    data, read back with a few lines of struct; and the prompt text of given token ids."""
    import struct
    import numpy as np
    import torch
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import reference_tools as ref
    import plain_llama as pl
    import tiny
    from cretif_b200.weights.random_model import write_random_model
    d = str(tmp_path / "m")
    write_random_model(d, dict(tiny.TINY_B, rope_interleaved=True), seed=22)
    path = str(tmp_path / "m.gguf")
    info = ref.write_gguf(d, path)
    raw = open(path, "rb").read()
    assert info["bytes"] == len(raw)
    magic, version, n_tensors, n_kv = struct.unpack_from("<IIQQ", raw, 0)
    assert (magic, version, n_kv) == (0x46554747, 3, 16)
    assert n_tensors == 3 + 9 * 3                     # embedding, norm, untied head, 3 layers
    at = 24

    def string():
        nonlocal at
        n, = struct.unpack_from("<Q", raw, at)
        at += 8 + n
        return raw[at - n:at].decode()

    def value(t):
        nonlocal at
        if t == 8:
            return string()
        if t == 9:
            et, n = struct.unpack_from("<IQ", raw, at)
            at += 12
            return [value(et) for _ in range(n)]
        fmt = {4: "<I", 6: "<f", 7: "<B"}[t]
        v, = struct.unpack_from(fmt, raw, at)
        at += struct.calcsize(fmt)
        return v
    meta = {}
    for _ in range(n_kv):
        key = string()
        t, = struct.unpack_from("<I", raw, at)
        at += 4
        meta[key] = value(t)
    assert meta["general.architecture"] == "llama" and meta["llama.block_count"] == 3
    assert meta["llama.attention.head_count_kv"] == 1 and meta["llama.vocab_size"] == 384
    assert abs(meta["llama.rope.freq_base"] - 100000.0) < 1e-3
    assert meta["tokenizer.ggml.merges"] == [] and meta["tokenizer.ggml.add_bos_token"] == 0
    tokens = meta["tokenizer.ggml.tokens"]
    ids = ref.char_ids(384)
    assert len(tokens) == 384 and len(set(tokens)) == 384 and len(ids) == 94
    text = ref.prompt_for([ids[3], ids[0], ids[93]], 384)
    assert [tokens.index(c) for c in text] == [ids[3], ids[0], ids[93]]
    tensors = {}
    for _ in range(n_tensors):
        name = string()
        nd, = struct.unpack_from("<I", raw, at)
        dims = struct.unpack_from(f"<{nd}Q", raw, at + 4)
        typ, off = struct.unpack_from("<IQ", raw, at + 4 + 8 * nd)
        at += 4 + 8 * nd + 12
        assert typ == 0 and off % 32 == 0
        tensors[name] = (dims, off)
    data = (at + 31) // 32 * 32
    _, w = pl.read_model_folder(d)
    dims, off = tensors["blk.2.attn_k.weight"]
    assert dims == (96, 32)                           # [in, out]: innermost first
    got = np.frombuffer(raw, dtype="<f4", count=96 * 32, offset=data + off).reshape(32, 96)
    assert np.array_equal(got, w["model.layers.2.self_attn.k_proj.weight"].float().numpy())
    assert "output.weight" in tensors and tensors["output_norm.weight"][0] == (96,)
