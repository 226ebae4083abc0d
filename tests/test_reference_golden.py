"""The reference engine's own output as the anchor.

``tests/golden/reference_*.json`` hold what the unmodified reference (its stock
``cuinfer <gguf> <prompt> --dump-logits``, src/main.cu:242-301) printed on an NVIDIA B200 for
seeded random models of this library written out as F32 GGUF files
(``tests/golden/make_reference_golden.py`` made them): the twenty largest logits at the last
position of a few prompts.  The model folders are made again here from the same
configuration and seed; a checksum makes sure they are the same weights.

On the CPU the plain implementation must reproduce those numbers (with the reference's
pairing of rotary channels, ``rope="interleaved"``), which pins every formula of
``tests/plain_llama.py`` to the reference's behaviour and not only to a reading of its source.
On the GPU the engine's own ``--dump-logits`` must print them too.
"""
import glob
import hashlib
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as pl

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLDEN = sorted(glob.glob(os.path.join(HERE, "golden", "reference_*.json")))
# The reference computes in float32 and prints six decimals; logits here are below 2.
ABS_TOL = 5e-5


def _sha256(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


@pytest.fixture(scope="module", params=GOLDEN, ids=[os.path.basename(p)[10:-5] for p in GOLDEN])
def golden(request, tmp_path_factory):
    from cretif_b200.weights.random_model import write_random_model
    with open(request.param) as f:
        doc = json.load(f)
    d = str(tmp_path_factory.mktemp("golden_model"))
    write_random_model(d, doc["config"], seed=doc["seed"])
    assert _sha256(os.path.join(d, "model.safetensors")) == doc["weights_sha256"], \
        "the random-weights mode no longer draws the weights the golden file was made with"
    return doc, d


def test_golden_files_exist():
    assert len(GOLDEN) >= 3


def _check_top(logits, top):
    """`top` is the reference's [(token id, logit)] in descending order."""
    logits = np.asarray(logits, dtype=np.float64)
    for tok, val in top:
        assert abs(logits[tok] - val) <= ABS_TOL, (tok, logits[tok], val)
    # the same twenty ids lead, up to ties within the tolerance
    ours = np.argsort(-logits)[:len(top)]
    floor = min(v for _, v in top)
    assert all(logits[t] >= floor - ABS_TOL for t in ours)
    assert int(np.argmax(logits)) == top[0][0] or abs(logits.max() - top[0][1]) <= ABS_TOL


def test_plain_implementation_reproduces_the_reference(golden):
    doc, d = golden
    cfg, w = pl.read_model_folder(d)
    assert cfg.get("rope_interleaved") is True
    for case in doc["cases"]:
        logits = pl.forward(cfg, w, case["ids"], rope="interleaved")[-1].numpy()
        _check_top(logits, case["top"])
    # the pairing matters: the other one gives other logits
    case = doc["cases"][-1]
    other = pl.forward(cfg, w, case["ids"], rope="half")[-1].numpy()
    assert max(abs(other[t] - v) for t, v in case["top"]) > 20 * ABS_TOL


@pytest.mark.gpu
def test_engine_dump_logits_reproduces_the_reference(golden, tmp_path):
    """python -m cretif_b200 <model> <ids> --dump-logits, in float32, as a user runs it."""
    doc, d = golden
    env = dict(os.environ, PYTHONPATH=ROOT)
    for i, case in enumerate(doc["cases"]):
        out = tmp_path / f"top{i}.json"
        proc = subprocess.run(
            [sys.executable, "-m", "cretif_b200", d, ",".join(str(t) for t in case["ids"]),
             "--dump-logits", str(out), "--dtype", "float32"],
            capture_output=True, text=True, env=env, timeout=900, cwd=ROOT)
        assert proc.returncode == 0, proc.stderr[-2000:]
        got = json.loads(out.read_text())
        assert got["num_input_tokens"] == len(case["ids"])
        ours = {e["token_id"]: e["logit_value"] for e in got["top_logits"]}
        for rank, (tok, val) in enumerate(case["top"]):
            if tok in ours:
                assert abs(ours[tok] - val) <= ABS_TOL, (tok, ours[tok], val)
            else:            # pushed out of the twenty by a tie within the tolerance
                assert val - min(ours.values()) <= ABS_TOL and rank >= 10
        assert abs(got["top_logits"][0]["logit_value"] - case["top"][0][1]) <= ABS_TOL
