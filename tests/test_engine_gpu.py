"""The engine against the plain implementation, in every way of cutting the work."""
import numpy as np
import pytest
import torch

import plain_llama
import tiny
from replay_cuts import (rel_err, run_batch, run_chunks, run_schedule, run_tail_by_one,
                         run_whole)

pytestmark = pytest.mark.gpu

# Relative to the largest plain logit.  float32: the library's contract.  bfloat16:
# activations and cached keys/values are rounded to 8 bits of mantissa (2^-9 relative
# each) several times a layer; sums and the residual stream stay in 32-bit.
TOL = {"float32": 1e-4, "bfloat16": 2e-2}
LENGTHS = {"A": [5, 9, 13, 70, 100], "B": [1, 17, 40, 130, 200], "C": [3, 33, 64, 65, 300],
           "W": [7, 24, 25, 90, 210]}


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_a_prompt_fed_in_chunks(engines, plain_logits, name, dtype):
    """A fourth cutting: several tokens at a cached position (the reference's forward takes
    any number of tokens at any position, src/attention.cu:60-77; its test is
    tests/test_attention.cu:307-336).  Alone, and inside a batch in which other sequences
    start fresh or go on by one token in the same step."""
    eng = engines(name, dtype)
    n = LENGTHS[name][3] + 30
    toks = tiny.tokens(name, n, 31)
    want = plain_logits(name, toks)
    assert rel_err(run_chunks(eng, toks, [40, 30, 1, 17]), want) <= TOL[dtype]
    assert rel_err(run_chunks(eng, toks, [1, 64, 2]), want) <= TOL[dtype]
    reqs = [toks, tiny.tokens(name, 50 + 17 + 3, 32), tiny.tokens(name, 9 + 4, 33),
            tiny.tokens(name, 66, 34)]
    rest = n - 40 - 30 - 1 - 17
    schedule = [[(0, 40)],
                [(0, 30), (1, 50)],                   # a chunk beside a fresh prompt
                [(0, 1), (1, 17), (2, 9)],            # one token, a chunk, a fresh prompt
                [(0, 17), (1, 1), (2, 1)],
                [(0, rest), (1, 1), (2, 1), (3, 66)],
                [(1, 1), (2, 1)],
                [(2, 1)]]
    for _ in range(2):                                # again: slots and blocks used again
        outs = run_schedule(eng, reqs, schedule)
        for r, got in zip(reqs, outs):
            assert rel_err(got, plain_logits(name, r)) <= TOL[dtype], len(r)
    eng.cache.check()
    assert eng.cache.stats()["slots_live"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sliding_window_from_config_json(engines, plain_logits, model_dirs, dtype):
    """`sliding_window` and `layer_types` in config.json: two of four layers see the last 24
    keys only.  Their cache group gives blocks back behind the window, the other keeps all.
    Small random weights give nearly uniform attention, so a key that is wrongly seen or
    wrongly hidden moves the logits little; the sharpened variant below makes it show."""
    eng = engines("W", dtype, max_tokens=1024)
    groups = eng.cache.stats()["groups"]
    assert sorted((g["window"], g["layers"]) for g in groups) == [(0, 2), (24, 2)]
    for n in LENGTHS["W"]:
        toks = tiny.tokens("W", n, 3)
        want = plain_logits("W", toks)
        assert rel_err(run_whole(eng, toks), want) <= TOL[dtype], n
        assert rel_err(run_tail_by_one(eng, toks, tail=32), want) <= TOL[dtype], n
    toks = tiny.tokens("W", 150, 4)
    assert rel_err(run_chunks(eng, toks, [30, 70, 1, 20]), plain_logits("W", toks)) <= TOL[dtype]
    reqs = [tiny.tokens("W", n + 10, 50 + n) for n in LENGTHS["W"][:4]]
    for _ in range(2):
        outs = run_batch(eng, reqs, LENGTHS["W"][:4])
        for r, got in zip(reqs, outs):
            assert rel_err(got, plain_logits("W", r)) <= TOL[dtype], len(r)
    eng.cache.check()
    # while a long sequence decodes, the window group holds two blocks, the other all four
    slot = eng.alloc_slot()
    eng.step([(slot, tiny.tokens("W", 200, 9))])
    free = dict(zip([g["window"] for g in groups], eng.cache.stats()["blocks_free"]))
    assert free[0] == eng.cache.n_blocks - 4 and free[24] == eng.cache.n_blocks - 2
    eng.free_slot(slot)
    eng.cache.check()


def test_a_sliding_window_with_sharp_attention(model_dirs, tmp_path):
    """Queries and keys of the two windowed layers scaled up (by 8: the scores by 64) so that
    every query reads a few particular keys: one key too many at the window's edge then moves
    the logits by 0.2 of the largest, fifty times what rounding to bfloat16 moves them."""
    import plain_llama as pl
    from cretif_b200.engine import Engine
    from cretif_b200.weights import write_model_folder
    cfg, w = pl.read_model_folder(model_dirs["W"])
    tensors = {k: v.to(torch.float32) for k, v in w.items()}
    for i in (0, 2):
        for name in ("q_proj", "k_proj"):
            tensors[f"model.layers.{i}.self_attn.{name}.weight"] *= 8.0
    d = str(tmp_path / "sharp_w")
    write_model_folder(d, cfg, tensors)
    cfg, w = pl.read_model_folder(d)
    toks = tiny.tokens("W", 140, 77)
    want = pl.forward(cfg, w, toks).numpy()
    wider = pl.forward(dict(cfg, sliding_window=25), w, toks).numpy()
    assert rel_err(wider, want) > 0.1                  # the edge matters with these weights
    eng = Engine(d, dtype="float32", max_tokens=512)
    assert rel_err(run_whole(eng, toks), want) <= 1e-4
    assert rel_err(run_tail_by_one(eng, toks, tail=40), want) <= 1e-4
    assert rel_err(run_chunks(eng, toks, [23, 24, 25, 1, 40]), want) <= 1e-4
    eng16 = Engine(d, dtype="bfloat16", max_tokens=512)
    want16 = pl.forward(cfg, w, toks, storage=torch.bfloat16).numpy()
    for got in (run_whole(eng16, toks), run_tail_by_one(eng16, toks, tail=40),
                run_chunks(eng16, toks, [23, 24, 25, 1, 40])):
        assert rel_err(got, want16) <= TOL["bfloat16"]  # against the plain model rounded alike
        assert rel_err(got, wider) > 0.1
