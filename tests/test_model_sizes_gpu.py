"""Layer sizes of the larger configurations (SmolLM2-360M and 1.7B), two layers each and a
small vocabulary: the kernels meet widths, head counts and feed-forward sizes that the tiny
configurations do not reach (15 heads on 5, 32 heads of their own, K = 8192)."""
import numpy as np
import pytest
import torch

import plain_llama as pl
from replay_cuts import rel_err, run_batch, run_tail_by_one, run_whole

pytestmark = pytest.mark.gpu

SIZES = {
    "360m": {"hidden_size": 960, "num_attention_heads": 15, "num_key_value_heads": 5,
             "intermediate_size": 2560, "rope_theta": 100000.0},
    "1.7b": {"hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 32,
             "intermediate_size": 8192, "rope_theta": 130000.0},
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from cretif_b200.weights.random_model import write_random_model
    out = {}
    for name, sizes in SIZES.items():
        cfg = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "vocab_size": 1000,
               "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
               "max_position_embeddings": 2048, **sizes}
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        write_random_model(d, cfg, seed=17)
        out[name] = (d, pl.read_model_folder(d))
    return out


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("name", ["360m", "1.7b"])
def test_larger_layer_sizes(folders, name, dtype, tol):
    from cretif_b200.engine import Engine
    d, (cfg, w) = folders[name]
    eng = Engine(d, dtype=dtype, max_tokens=2048)
    rng = np.random.default_rng(5)
    reqs = [rng.integers(0, 1000, size=n).tolist() for n in (150, 40, 9)]
    wants = [pl.forward(cfg, w, r).numpy() for r in reqs]
    assert rel_err(run_whole(eng, reqs[0]), wants[0]) <= tol            # tensor-core prefill
    assert rel_err(run_tail_by_one(eng, reqs[1], tail=8), wants[1]) <= tol
    outs = run_batch(eng, reqs, [140, 33, 2])                            # then decode together
    for got, want in zip(outs, wants):
        assert rel_err(got, want) <= tol
    eng.cache.check()
