"""The sizes and the regime that bench.py times, compared with the plain model.

* SmolLM2-135M as the preset gives it — 30 layers, width 576, 9 heads on 3 key/value heads,
  feed-forward 1536, vocabulary 49,152, tied head — on short requests in every cutting:
  float32 within 1e-4, bfloat16 within 2e-2 of the largest plain logit.
* The same layer sizes with two layers and a small vocabulary where the plain model is
  affordable on long inputs: a 2,048-token prompt, batches of 8 and 40 prompts of unequal
  lengths 256..2,048 followed by decode steps whose contexts cross 2,048, decode batches of
  16, 33 and 64 through ``Engine.step`` and through ``generate``.

The last test checks, from the kernels' own launch counts, that every variant bench.py's
numbers come from (row groups, shared norm prologue, streaming ring, the cluster merge
of the decode attention, the persistent tensor-core product, the tensor-core prefill
attention with a CTA's two groups of warps on one query tile and on two) ran under one of
these comparisons.
"""
import numpy as np
import pytest
import torch

import plain_llama as pl
from replay_cuts import rel_err, run_batch, run_chunks, run_tail_by_one, run_whole

pytestmark = pytest.mark.gpu
TOL = {"float32": 1e-4, "bfloat16": 2e-2}
WIDE = {"architectures": ["LlamaForCausalLM"], "hidden_size": 576, "num_hidden_layers": 2,
        "num_attention_heads": 9, "num_key_value_heads": 3, "head_dim": 64,
        "intermediate_size": 1536, "vocab_size": 1000, "rope_theta": 100000.0,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 4096}
_counts_at_start = {}


@pytest.fixture(scope="module", autouse=True)
def _variant_counts_at_start():
    from cretif_b200.csrc import ops
    _counts_at_start.update(ops.variant_counts())
    yield


@pytest.fixture(scope="module")
def full_model(tmp_path_factory):
    from cretif_b200.config import preset
    from cretif_b200.weights.random_model import write_random_model
    d = str(tmp_path_factory.mktemp("smollm2_135m"))
    write_random_model(d, preset("smollm2-135m"), seed=1234)
    return d, pl.read_model_folder(d)


@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    """135M layer sizes, two layers; layer 0's queries and keys are scaled up so that a query
    reads particular keys, far ones among them (random weights alone give nearly uniform
    attention, under which a wrong key hides)."""
    from cretif_b200.weights import write_model_folder
    from cretif_b200.weights.random_model import write_random_model
    flat = str(tmp_path_factory.mktemp("wide_flat"))
    write_random_model(flat, WIDE, seed=77)
    cfg, w = pl.read_model_folder(flat)
    tensors = {k: v.to(torch.bfloat16) for k, v in w.items()}
    for name in ("q_proj", "k_proj"):
        key = f"model.layers.0.self_attn.{name}.weight"
        tensors[key] = (w[key] * 5.0).to(torch.bfloat16)
    d = str(tmp_path_factory.mktemp("wide"))
    write_model_folder(d, cfg, tensors)
    return d, pl.read_model_folder(d)


@pytest.fixture(scope="module")
def wide_engines(wide_model):
    from cretif_b200.engine import Engine
    made = {}

    def get(dtype, max_tokens):
        if (dtype, max_tokens) not in made:
            made[(dtype, max_tokens)] = Engine(wide_model[0], dtype=dtype, max_tokens=max_tokens)
        return made[(dtype, max_tokens)]
    return get


def _plain(model, toks, dtype):
    cfg, w = model[1]
    storage = torch.bfloat16 if dtype == "bfloat16" else None
    return pl.forward(cfg, w, list(toks), storage=storage).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_smollm2_135m_at_full_depth_in_every_cutting(full_model, dtype):
    from cretif_b200.engine import Engine
    d, (cfg, w) = full_model
    assert (cfg["num_hidden_layers"], cfg["vocab_size"], cfg["hidden_size"]) == (30, 49152, 576)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    rng = np.random.default_rng(135)
    reqs = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in (70, 9, 33)]
    wants = [pl.forward(cfg, w, r).numpy() for r in reqs]
    tol = TOL[dtype]
    assert rel_err(run_whole(eng, reqs[0]), wants[0]) <= tol
    assert rel_err(run_tail_by_one(eng, reqs[0], tail=32), wants[0]) <= tol
    assert rel_err(run_chunks(eng, reqs[0], [40, 20]), wants[0]) <= tol
    for _ in range(2):
        for got, want in zip(run_batch(eng, reqs, [60, 5, 20]), wants):
            assert rel_err(got, want) <= tol
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_of_2048_tokens(wide_model, wide_engines, dtype):
    eng = wide_engines(dtype, 8 * 4096)
    toks = np.random.default_rng(1).integers(0, 1000, size=2048).tolist()
    want = _plain(wide_model, toks, dtype)
    got = run_whole(eng, toks)
    assert got.shape == (2048, 1000)
    assert rel_err(got, want) <= TOL[dtype]
    if dtype == "bfloat16":          # the last 40 tokens one by one, contexts of 2,008 and more
        assert rel_err(run_tail_by_one(eng, toks, tail=40), want) <= TOL[dtype]


def _prefill_then_decode(eng, requests, prompt_lens, rows_of):
    """Prompts of unequal lengths in one step (logits at ``rows_of(length)``), then one token
    each per step until each request's tokens run out; returns (request, place, logits)."""
    slots = [eng.alloc_slot() for _ in requests]
    out = []
    try:
        wants = [rows_of(p) for p in prompt_lens]
        logits = eng.step([(s, r[:p]) for s, r, p in zip(slots, requests, prompt_lens)],
                          wants).cpu().numpy()
        o = 0
        for r, rows in enumerate(wants):
            for place in rows:
                out.append((r, place, logits[o]))
                o += 1
        fed = list(prompt_lens)
        live = list(range(len(requests)))
        while live:
            live = [r for r in live if fed[r] < len(requests[r])]
            if not live:
                break
            logits = eng.step([(slots[r], [requests[r][fed[r]]]) for r in live], "all"
                              ).cpu().numpy()
            for i, r in enumerate(live):
                out.append((r, fed[r], logits[i]))
                fed[r] += 1
        return out
    finally:
        for s in slots:
            eng.free_slot(s)


@pytest.mark.parametrize("batch,lengths", [
    (8, [2048, 2041, 1500, 1024, 700, 513, 300, 256]),
    (40, None)])
def test_batches_of_unequal_prompts_then_decoding_past_2048(wide_model, wide_engines, batch,
                                                            lengths):
    dtype = "bfloat16"
    eng = wide_engines(dtype, 40 * 2112)
    rng = np.random.default_rng(batch)
    if lengths is None:
        lengths = [2048, 2046, 2040] + rng.integers(256, 2049, size=batch - 3).tolist()
    steps = 10
    requests = [rng.integers(0, 1000, size=n + steps).tolist() for n in lengths]
    # every place of the small batch; every 97th and the last two of each prompt of the large
    rows_of = (lambda p: list(range(p))) if batch == 8 else \
        (lambda p: sorted(set(range(0, p, 97)) | {p - 2, p - 1}))
    got = _prefill_then_decode(eng, requests, lengths, rows_of)
    plain = [_plain(wide_model, r, dtype) for r in requests]
    scale = max(float(np.abs(p).max()) for p in plain)
    worst = max(float(np.abs(row.astype(np.float64) - plain[r][place]).max())
                for r, place, row in got)
    assert worst / scale <= TOL[dtype]
    assert sum(1 for r, place, _ in got if place >= 2048) >= 3 * (steps - 8)
    eng.cache.check()
    assert eng.cache.stats()["slots_live"] == 0


def test_a_repeated_step_of_16384_tokens_is_replayed_as_a_graph(wide_model, wide_engines):
    """Eight prompts of 2,048 tokens in one step, three times with the same tokens in other
    slots: the first runs eagerly, the second is captured, the third is the graph's replay;
    all three give the same logits, and those of the first prompt are the plain model's."""
    eng = wide_engines("bfloat16", 40 * 2112)
    rng = np.random.default_rng(16384)
    prompts = [rng.integers(0, 1000, size=2048).tolist() for _ in range(8)]
    key = (tuple(2048 for _ in prompts), "last", 0)
    runs = []
    for i in range(3):
        spare = [eng.alloc_slot() for _ in range(i)]       # so that the slots differ each time
        slots = [eng.alloc_slot() for _ in prompts]
        runs.append(eng.step(list(zip(slots, prompts)), "last").cpu().numpy())
        assert (key in eng._graphs) == (i >= 1)
        for s in slots + spare:
            eng.free_slot(s)
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    want = _plain(wide_model, prompts[0], "bfloat16")[-1]
    assert rel_err(runs[2][0], want) <= TOL["bfloat16"]
    eng.cache.check()


@pytest.mark.parametrize("batch", [16, 33, 64])
def test_decode_batches_through_the_step_function(wide_model, wide_engines, batch):
    """Short unequal prompts, four of them long enough that the decode attention is planned
    for contexts beyond 2,048 as in the benchmark; then eight tokens each."""
    dtype = "bfloat16"
    eng = wide_engines(dtype, 40 * 2112)
    rng = np.random.default_rng(100 + batch)
    lengths = [2047, 2050, 1100, 600] + rng.integers(5, 70, size=batch - 4).tolist()
    requests = [rng.integers(0, 1000, size=n + 8).tolist() for n in lengths]
    got = _prefill_then_decode(eng, requests, lengths, lambda p: [p - 1])
    plain = [_plain(wide_model, r, dtype) for r in requests]
    scale = max(float(np.abs(p).max()) for p in plain)
    worst = max(float(np.abs(row.astype(np.float64) - plain[r][place]).max())
                for r, place, row in got)
    assert worst / scale <= TOL[dtype]
    eng.cache.check()


@pytest.mark.parametrize("batch", [16, 33, 64])
def test_decode_batches_through_generate(wide_model, wide_engines, batch):
    """Greedy generation of a whole batch.  float32: the plain model's tokens.  bfloat16:
    every chosen token is, by the plain model rounded alike and fed the same tokens, the best
    one or within the bound of the best (near ties may fall either way)."""
    cfg, w = wide_model[1]
    rng = np.random.default_rng(200 + batch)
    prompts = [rng.integers(0, 1000, size=n).tolist()
               for n in rng.integers(3, 40, size=batch).tolist()]
    eng32 = wide_engines("float32", 8 * 4096)
    got = eng32.generate(prompts, max_tokens=5, stop_ids=[], max_batch=batch)
    for p, r in zip(prompts[:: max(1, batch // 8)], got[:: max(1, batch // 8)]):
        assert r.tokens == pl.greedy(cfg, w, p, 5)
    eng16 = wide_engines("bfloat16", 40 * 2112)
    got16 = eng16.generate(prompts, max_tokens=5, stop_ids=[], max_batch=batch)
    for p, r in zip(prompts, got16):
        assert len(r.tokens) == 5
        logits = _plain(wide_model, p + r.tokens[:-1], "bfloat16")[len(p) - 1:]
        bound = 2 * TOL["bfloat16"] * float(np.abs(logits).max())
        for row, tok in zip(logits, r.tokens):
            assert row.max() - row[tok] <= bound
    eng16.cache.check()
    assert eng16.cache.stats()["slots_live"] == 0


def test_every_path_the_benchmark_times_was_compared():
    """The tests above ran these kernel variants (counted by the launchers themselves)."""
    from cretif_b200.csrc import ops
    now = ops.variant_counts()
    ran = {k for k, v in now.items() if v > _counts_at_start.get(k, 0)}
    needed = {"fused_registers", "fused_row_groups", "fused_cluster2", "fused_cluster4",
              "stream", "stream_row_groups", "decode_cluster", "prefill_attn_split",
              "prefill_attn_pair", "tc64", "tc128", "tc192", "tc_several_tiles"}
    assert needed <= ran, sorted(needed - ran)
