"""The engine against the plain implementation, in every way of cutting the work."""
import numpy as np
import pytest
import torch

import plain_llama
import tiny
from replay_cuts import rel_err, run_batch, run_tail_by_one, run_whole

pytestmark = pytest.mark.gpu

# Relative to the largest plain logit.  float32: the library's contract.  bfloat16:
# activations and cached keys/values are rounded to 8 bits of mantissa (2^-9 relative
# each) several times a layer; sums and the residual stream stay in 32-bit.
TOL = {"float32": 1e-4, "bfloat16": 2e-2}
LENGTHS = {"A": [5, 9, 13, 70, 100], "B": [1, 17, 40, 130, 200], "C": [3, 33, 64, 65, 300]}


@pytest.fixture(scope="module")
def engines(model_dirs):
    from cretif_b200.engine import Engine
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(model_dirs[name], dtype=dtype, max_tokens=max_tokens)
        return made[key]
    return get


@pytest.fixture(scope="module")
def plain_logits(plain_models):
    memo = {}

    def get(name, toks):
        key = (name, tuple(toks))
        if key not in memo:
            cfg, w = plain_models[name]
            memo[key] = plain_llama.forward(cfg, w, list(toks)).numpy()
        return memo[key]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_each_request_whole(engines, plain_logits, name, dtype):
    eng = engines(name, dtype)
    for n in LENGTHS[name]:
        toks = tiny.tokens(name, n, 1)
        got = run_whole(eng, toks)
        assert got.shape == (n, eng.vocab_size)
        assert rel_err(got, plain_logits(name, toks)) <= TOL[dtype], (name, n)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_tokens_one_by_one(engines, plain_logits, name, dtype):
    eng = engines(name, dtype)
    for n in LENGTHS[name]:
        toks = tiny.tokens(name, n, 2)
        got = run_tail_by_one(eng, toks, tail=32)
        assert rel_err(got, plain_logits(name, toks)) <= TOL[dtype], (name, n)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_reuse_slots(engines, plain_logits, name, dtype):
    """Batches of unequal lengths, one after another, on a cache too small to hold two
    batches at once, so that blocks and slots of the first are used again."""
    eng = engines(name, dtype, max_tokens=512)
    lens = LENGTHS[name]
    for round_ in range(3):
        reqs = [tiny.tokens(name, n + 8 + 3 * i, 10 + round_) for i, n in enumerate(lens[:4])]
        prompts = [min(lens[i], len(r)) for i, r in enumerate(reqs)]
        outs = run_batch(eng, reqs, prompts)
        for r, got in zip(reqs, outs):
            assert rel_err(got, plain_logits(name, r)) <= TOL[dtype], (name, round_, len(r))
        eng.cache.check()
        assert eng.cache.stats()["slots_live"] == 0


@pytest.mark.parametrize("name", ["A", "C"])
def test_bfloat16_without_the_fused_few_token_kernels(engines, plain_logits, name):
    """The separate norm / product / rotary / activation kernels serve steps the fused ones
    refuse; switched to by hand here, they give the same logits within the same bound."""
    from cretif_b200.parts.attention import enable_fused_steps
    eng = engines(name, "bfloat16")
    toks = tiny.tokens(name, LENGTHS[name][3] + 5, 9)
    fused = run_tail_by_one(eng, toks, tail=32)
    enable_fused_steps(False)
    try:
        plain = run_tail_by_one(eng, toks, tail=32)
    finally:
        enable_fused_steps(True)
    want = plain_logits(name, toks)
    assert rel_err(fused, want) <= TOL["bfloat16"] and rel_err(plain, want) <= TOL["bfloat16"]
    assert rel_err(fused, plain) <= TOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_repeated_step_shape_is_replayed_as_a_graph(model_dirs, plain_logits, dtype):
    """The first step of a shape runs eagerly, the second is captured, later ones are
    replayed: other tokens, other slots and other cache blocks each time, same logits as the
    plain model; and an engine without captured steps agrees."""
    from cretif_b200.engine import Engine
    eng = Engine(model_dirs["B"], dtype=dtype, max_tokens=1024)
    off = Engine(model_dirs["B"], dtype=dtype, max_tokens=1024, step_graphs=False)
    assert eng.step_graphs and not off.step_graphs
    held = [eng.alloc_slot() for _ in range(2)]           # shift the slots the runs will get
    for i in range(5):
        toks = tiny.tokens("B", 70, 100 + i)
        got = run_tail_by_one(eng, toks, tail=6)          # shapes (64,) and (1,) repeat
        assert rel_err(got, plain_logits("B", toks)) <= TOL[dtype], i
        if i == 2:
            eng.free_slot(held.pop())                      # and change them again
    assert len(eng._graphs) == 2
    toks = tiny.tokens("B", 70, 104)
    assert rel_err(run_tail_by_one(off, toks, tail=6), plain_logits("B", toks)) <= TOL[dtype]
    assert len(off._graphs) == 0
    # batches: the shape is the tuple of lengths
    reqs = [tiny.tokens("B", n, 200 + n) for n in (30, 9, 17)]
    for _ in range(3):
        outs = run_batch(eng, reqs, [25, 9, 12])
        for r, got in zip(reqs, outs):
            assert rel_err(got, plain_logits("B", r)) <= TOL[dtype]
    eng.cache.check()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_whole_step_kernel_equals_the_kernels_of_the_parts(engines, plain_logits, name):
    """Decode steps of few sequences can run as one persistent launch (switched on here); by
    default they run through the parts' kernels.  Both are compared with the plain model and
    with each other."""
    from cretif_b200.engine import step_kernel
    eng = engines(name, "bfloat16")
    assert eng.model.step_kernel.ok, eng.model.step_kernel.reason
    reqs = [tiny.tokens(name, n + 20, 60 + i) for i, n in enumerate(LENGTHS[name][:4])]
    prompts = [len(r) - 20 for r in reqs]
    without = run_batch(eng, reqs, prompts)
    step_kernel.enable(True)
    try:
        with_kernel = run_batch(eng, reqs, prompts)
    finally:
        step_kernel.enable(False)
    for r, a, b in zip(reqs, with_kernel, without):
        want = plain_logits(name, r)
        assert rel_err(a, want) <= TOL["bfloat16"] and rel_err(b, want) <= TOL["bfloat16"]
        assert rel_err(a, b) <= TOL["bfloat16"]
    eng.cache.check()
