#!/usr/bin/env python3
"""Makes the golden files of this folder by running the UNMODIFIED reference engine.

    python baseline/reference_tools.py build <directory of the reference>   # once, needs nvcc
    python tests/golden/make_reference_golden.py                            # on a GPU

For each model below a folder with seeded random weights is written (this library's
random-weights mode, ``rope_interleaved: true`` because the reference rotates pairs
(2j, 2j+1) of the rows as stored), exported as an F32 GGUF file, and the reference's stock
``cuinfer <gguf> <prompt> --dump-logits`` (src/main.cu:242-301) is run on a few prompts.  Its
output — the twenty largest logits at the last position — is stored with the prompt's token
ids, the configuration, the seed and a checksum of the weights in ``reference_<name>.json``.

``tests/test_reference_golden.py`` then checks, on the CPU, that the plain implementation
reproduces these numbers, and on the GPU that the engine's own ``--dump-logits`` does.
Nothing here is needed to run those tests; the script is kept so that the files can be made
again.
"""
import hashlib
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))
sys.path.insert(0, os.path.dirname(HERE))

import reference_tools as ref  # noqa: E402
import tiny  # noqa: E402
from cretif_b200.config import preset  # noqa: E402
from cretif_b200.weights.random_model import write_random_model  # noqa: E402

MODELS = {
    "tiny_a": (dict(tiny.TINY_A, rope_interleaved=True), 11, [1, 7, 40, 100]),
    "tiny_b": (dict(tiny.TINY_B, rope_interleaved=True), 22, [3, 64, 65, 200]),
    "smollm2_135m": (dict(preset("smollm2-135m"), rope_interleaved=True), 1234, [33]),
}


def file_sha256(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def main():
    why = ref.available()
    if why:
        sys.exit(why)
    for name, (cfg, seed, lengths) in MODELS.items():
        with tempfile.TemporaryDirectory(prefix="cretif_golden_") as tmp:
            write_random_model(tmp, cfg, seed=seed)
            gguf = os.path.join(tmp, "model.gguf")
            ref.write_gguf(tmp, gguf)
            V = cfg["vocab_size"]
            chars = ref.char_ids(V)
            rng = np.random.default_rng(seed)
            cases = []
            for n in lengths:
                ids = [chars[i] for i in rng.integers(0, len(chars), size=n)]
                doc = ref.dump_logits(gguf, ref.prompt_for(ids, V), os.path.join(tmp, "o.json"))
                assert doc["input_token_ids"] == ids, "the prompt did not encode as planned"
                cases.append({"ids": ids,
                              "top": [[e["token_id"], e["logit_value"]] for e in doc["top_logits"]]})
            out = {"made_by": "tests/golden/make_reference_golden.py with the reference's stock "
                              "`cuinfer --dump-logits` on an NVIDIA B200",
                   "config": cfg, "seed": seed,
                   "weights_sha256": file_sha256(os.path.join(tmp, "model.safetensors")),
                   "cases": cases}
        path = os.path.join(HERE, f"reference_{name}.json")
        with open(path, "w") as f:
            json.dump(out, f, indent=1)
            f.write("\n")
        print(f"wrote {path}: {len(cases)} prompts")


if __name__ == "__main__":
    main()
