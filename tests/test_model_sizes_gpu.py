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


def test_a_large_step_at_360m_sizes_takes_the_two_cta_products(folders):
    """Four prompts of 2,048 tokens in one step at SmolLM2-360M layer sizes: enough tiles and
    a long enough K that gate|up and the down projection run with two CTAs on a tile
    (cta_group::2).  The last positions of every prompt and every 97th of the first against the
    plain model rounded alike."""
    from cretif_b200.csrc import ops
    from cretif_b200.engine import Engine
    d, (cfg, w) = folders["360m"]
    eng = Engine(d, dtype="bfloat16", max_tokens=4 * 2112)
    rng = np.random.default_rng(360)
    prompts = [rng.integers(0, 1000, size=2048).tolist() for _ in range(4)]
    rows = [sorted(set(range(0, 2048, 97)) | {2047})] + [[2047]] * 3
    before = ops.variant_counts()["tc_pair"]
    slots = [eng.alloc_slot() for _ in prompts]
    got = eng.step(list(zip(slots, prompts)), rows).cpu().numpy()
    for s_ in slots:
        eng.free_slot(s_)
    assert ops.variant_counts()["tc_pair"] >= before + 4          # two layers, two products each
    first = pl.forward(cfg, w, prompts[0], storage=torch.bfloat16).numpy()
    n0 = len(rows[0])
    assert rel_err(got[:n0], first[rows[0]]) <= 2e-2
    for b in (1, 2, 3):
        want = pl.forward(cfg, w, prompts[b], storage=torch.bfloat16).numpy()[-1]
        assert rel_err(got[n0 + b - 1], want) <= 2e-2
    eng.cache.check()
