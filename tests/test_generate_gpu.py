"""Generation through the Python entry point, long decoding, first tokens, reused slots,
sharpened attention, sampling and the replay program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as pl
import tiny
from replay_cuts import rel_err, run_batch, run_tail_by_one, run_whole

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 1e-4, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def engines(model_dirs):
    from cretif_b200.engine import Engine
    made = {}

    def get(name, dtype, max_tokens=2048):
        if (name, dtype, max_tokens) not in made:
            made[(name, dtype, max_tokens)] = Engine(model_dirs[name], dtype=dtype,
                                                     max_tokens=max_tokens)
        return made[(name, dtype, max_tokens)]
    return get


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_plain_in_float32(engines, plain_models, name):
    eng = engines(name, "float32")
    cfg, w = plain_models[name]
    prompts = [tiny.tokens(name, n, 20 + n) for n in (1, 6, 19, 70)]
    got = eng.generate(prompts, max_tokens=9, stop_ids=[])
    for p, r in zip(prompts, got):
        assert r.tokens == pl.greedy(cfg, w, p, 9) and r.finish_reason == "length"
    # the same requests without CUDA graphs, and one at a time, give the same tokens
    again = eng.generate(prompts, max_tokens=9, stop_ids=[], use_graph=False)
    assert [r.tokens for r in again] == [r.tokens for r in got]
    for p, r in zip(prompts, got):
        assert eng.generate([p], max_tokens=9, stop_ids=[])[0].tokens == r.tokens
    eng.cache.check()
    assert eng.cache.stats()["slots_live"] == 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_in_bfloat16_picks_near_best_tokens(engines, plain_models, name):
    """bfloat16 may break near-ties differently, so every generated token is checked against
    the plain logits of its own prefix: it must be within tolerance of the best."""
    eng = engines(name, "bfloat16")
    cfg, w = plain_models[name]
    prompts = [tiny.tokens(name, n, 30 + n) for n in (3, 33, 80)]
    got = eng.generate(prompts, max_tokens=12, stop_ids=[])
    for p, r in zip(prompts, got):
        assert len(r.tokens) == 12
        logits = pl.forward(cfg, w, p + r.tokens[:-1])[len(p) - 1:]
        for t, row in zip(r.tokens, logits):
            assert row.max() - row[t] <= TOL["bfloat16"] * row.abs().max()


def test_stop_tokens_end_a_sequence_and_are_kept(engines, plain_models):
    eng = engines("A", "float32")
    cfg, w = plain_models["A"]
    prompts = [tiny.tokens("A", n, 40 + n) for n in (5, 9, 13)]
    free = pl.greedy(cfg, w, prompts[1], 8)
    stop = free[3]
    got = eng.generate(prompts, max_tokens=8, stop_ids=[stop])
    first = free.index(stop)
    assert got[1].tokens == free[:first + 1] and got[1].finish_reason == "stop"
    for p, r in zip(prompts, got):
        want = pl.greedy(cfg, w, p, 8, stop_ids={stop})
        assert r.tokens == want
    # the model's own eos_token_id is the default stop set
    assert eng.spec.stop_token_ids == [7]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_one_step_ahead_of_the_host_changes_no_token(engines, dtype):
    """The backend launches the next decode step before it hands a step's tokens to the
    loop.  Sequences that end on a stop token, at different times, are in the step in flight:
    their part is dropped, their slots come back afterwards, the others' tokens are the same
    as without running ahead, and no slot is lost."""
    from cretif_b200.engine.generate import EngineBackend, GenerationLoop
    from cretif_b200.sampling import SamplingParams
    eng = engines("B", dtype)
    prompts = [tiny.tokens("B", n, 70 + n) for n in (4, 11, 7, 19, 2)]

    def run(ahead, stops, max_tokens):
        be = EngineBackend(eng, SamplingParams(), use_graph=True, run_ahead=ahead)
        loop = GenerationLoop(be, stops, eng.cache.max_tokens, eng.cache.max_len,
                              eng.cache.block_tokens, max_batch=4)     # two batches
        out = loop.run(prompts, max_tokens)
        assert eng.cache.stats()["slots_live"] == 0
        eng.cache.check()
        return [(r.tokens, r.finish_reason) for r in out]

    free = run(False, [], 24)
    # stop tokens that some sequences meet early, some late and some never
    stops = {free[0][0][5], free[2][0][14], free[3][0][1]}
    plain = run(False, stops, 24)
    assert any(reason == "stop" for _, reason in plain) and any(r == "length" for _, r in plain)
    assert len({len(t) for t, _ in plain}) > 2
    assert run(True, stops, 24) == plain
    assert run(True, [], 24) == free
    # a sequence that fills its reservation exactly is not stepped beyond it
    assert run(True, stops, 3) == run(False, stops, 3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(engines, plain_models, dtype):
    """300 tokens fed one by one after a short prompt (crossing four cache blocks)."""
    eng = engines("C", dtype)
    cfg, w = plain_models["C"]
    toks = tiny.tokens("C", 320, 5)
    got = run_tail_by_one(eng, toks, tail=300)
    assert rel_err(got, pl.forward(cfg, w, toks).numpy()) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(engines, plain_models, name, dtype):
    """One-token prompts, alone and in a batch, then the next tokens one by one."""
    eng = engines(name, dtype)
    cfg, w = plain_models[name]
    reqs = [tiny.tokens(name, 6, 50 + i) for i in range(3)]
    wants = [pl.forward(cfg, w, r).numpy() for r in reqs]
    assert rel_err(run_tail_by_one(eng, reqs[0], tail=5), wants[0]) <= TOL[dtype]
    outs = run_batch(eng, reqs, [1, 1, 2])
    for got, want in zip(outs, wants):
        assert rel_err(got, want) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_reused_slot_shows_nothing_of_its_last_owner(engines, plain_models, dtype):
    eng = engines("B", dtype, max_tokens=256)
    cfg, w = plain_models["B"]
    long_req, short_req = tiny.tokens("B", 200, 60), tiny.tokens("B", 30, 61)
    alone = run_whole(eng, short_req)
    run_whole(eng, long_req)                       # fills the slot and blocks, then frees them
    after = run_tail_by_one(eng, short_req, tail=20)
    assert rel_err(after, pl.forward(cfg, w, short_req).numpy()) <= TOL[dtype]
    assert rel_err(after, alone) <= TOL[dtype]


# name -> (gain of layer 0's query and key projections, tokens of the long request)
SHARP = {"A": (32.0, 120), "B": (24.0, 250), "C": (24.0, 300)}


@pytest.fixture(scope="module")
def sharp_models(tmp_path_factory, model_dirs):
    """Every tiny configuration with layer 0's query and key projections scaled up so that
    attention is sharp: each query then reads a few particular keys, far ones included, and a
    wrong key, position or cache slot changes the logits visibly (head sizes 16, 32 and 48,
    both pairings of the rotary channels)."""
    from safetensors import safe_open
    from cretif_b200.weights import write_model_folder
    made = {}
    for name, (gain, _) in SHARP.items():
        d = str(tmp_path_factory.mktemp(f"model_{name}_sharp"))
        tensors = {}
        with safe_open(os.path.join(model_dirs[name], "model.safetensors"), framework="pt") as f:
            for k in f.keys():
                tensors[k] = f.get_tensor(k)
        for proj in ("q_proj", "k_proj"):
            key = f"model.layers.0.self_attn.{proj}.weight"
            tensors[key] = (tensors[key].float() * gain).to(torch.bfloat16)
        with open(os.path.join(model_dirs[name], "config.json")) as f:
            cfg = json.load(f)
        write_model_folder(d, cfg, tensors)
        made[name] = (d, pl.read_model_folder(d))
    return made


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_sharp_attention_over_hundreds_of_keys(sharp_models, name, dtype):
    from cretif_b200.engine import Engine
    d, (cfg, w) = sharp_models[name]
    n = SHARP[name][1]
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    # With scores this large, rounding q and k to bfloat16 alone moves the softmax by more
    # than the usual bound, in any engine; so the bfloat16 run is compared with the plain
    # model rounded at the same stores.  float32 is compared with the exact plain model.
    storage = torch.bfloat16 if dtype == "bfloat16" else None
    plain = lambda t: pl.forward(cfg, w, t, storage=storage).numpy()
    toks = tiny.tokens(name, n, 70)
    want = plain(toks)
    exact = pl.forward(cfg, w, toks).numpy()
    if storage is not None:      # the sharpening bites: plain rounding alone breaks the bound
        assert rel_err(want, exact) > TOL[dtype]
    assert rel_err(run_whole(eng, toks), want) <= TOL[dtype]
    assert rel_err(run_tail_by_one(eng, toks, tail=32), want) <= TOL[dtype]
    reqs = [toks, tiny.tokens(name, 2 * n // 5, 71), tiny.tokens(name, 3 * n // 4, 72)]
    outs = run_batch(eng, reqs, [n - 32, 2 * n // 7, 1])
    for r, got in zip(reqs, outs):
        assert rel_err(got, plain(r)) <= TOL[dtype]
    eng.cache.check()


def test_sampling_through_the_entry_point(engines):
    eng = engines("A", "float32")
    prompts = [tiny.tokens("A", n, 80 + n) for n in (4, 11, 30)]
    a = eng.generate(prompts, max_tokens=10, temperature=1.5, seed=5, stop_ids=[])
    b = eng.generate(prompts, max_tokens=10, temperature=1.5, seed=5, stop_ids=[])
    c = eng.generate(prompts, max_tokens=10, temperature=1.5, seed=6, stop_ids=[])
    assert [r.tokens for r in a] == [r.tokens for r in b]
    assert [r.tokens for r in a] != [r.tokens for r in c]
    # request 0's draws do not depend on who shares its batch
    alone = eng.generate(prompts[:1], max_tokens=10, temperature=1.5, seed=5, stop_ids=[])
    assert alone[0].tokens == a[0].tokens
    k1 = eng.generate(prompts, max_tokens=6, temperature=0.7, top_k=1, stop_ids=[])
    g = eng.generate(prompts, max_tokens=6, stop_ids=[])
    assert [r.tokens for r in k1] == [r.tokens for r in g]
    with pytest.raises(ValueError):
        eng.generate(prompts, top_k=-1)


def test_step_refuses_what_it_cannot_run(engines):
    from cretif_b200.cache import CacheError, CacheFull
    from cretif_b200.engine import StepError
    eng = engines("A", "float32")
    s = eng.alloc_slot()
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([(s, [1, 256])])
    with pytest.raises(StepError, match="at least one token"):
        eng.step([(s, [])])
    with pytest.raises(CacheError):
        eng.step([(s, [1]), (s, [2])])
    with pytest.raises(CacheFull, match="longest"):
        eng.step([(s, [1] * 129)])
    assert eng.cache.length(s) == 0                  # refused steps left nothing behind
    eng.step([(s, [1, 2, 3])])
    t = eng.alloc_slot()
    # a sequence that goes on beside one that starts is an ordinary step
    assert tuple(eng.step([(s, [4]), (t, [1, 2])], "all").shape) == (3, 256)
    with pytest.raises(StepError, match="wanted places"):
        eng.step([(s, [4])], want=[[1]])
    assert tuple(eng.step([(s, [4])], want=[[]]).shape) == (0, 256)
    eng.free_slot(s); eng.free_slot(t)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, plain_models, tmp_path, dtype):
    """bin/trace_run as a user runs it: steps on stdin, logits files out, `done` lines."""
    cfg, w = plain_models["B"]
    ra, rb, rc = (tiny.tokens("B", n, 90 + n) for n in (40, 9, 70))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ra[:38], "want": [0, 37]},
                                     {"id": "b", "tokens": rb[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [ra[38]], "want": [0]},
                                     {"id": "b", "tokens": [rb[8]], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [ra[39]], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": rc[:30], "want": list(range(30))}],
              "end": []},
             # a further chunk of c beside a request that starts
             {"step": 4, "entries": [{"id": "c", "tokens": rc[30:], "want": list(range(40))},
                                     {"id": "d", "tokens": rb, "want": [8]}],
              "end": ["c", "d"]}]
    out = tmp_path / "out"
    env = dict(os.environ, PYTHONPATH="")
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["B"],
         "--dtype", dtype, "--out", str(out), "--max-tokens", "192"],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
        env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "4"]
    V = cfg["vocab_size"]
    la, lb, lc = (pl.forward(cfg, w, r).numpy() for r in (ra, rb, rc))
    read = lambda i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
    tol = TOL[dtype]
    got0 = read(0)
    assert got0.shape == (3, V)
    assert rel_err(got0, np.stack([la[0], la[37], lb[7]])) <= tol
    assert rel_err(read(1), la[38:39]) <= tol
    assert rel_err(read(2), la[39:40]) <= tol
    assert rel_err(read(3), lc[:30]) <= tol
    assert rel_err(read(4), np.concatenate([lc[30:], lb[8:9]])) <= tol


def test_command_line(model_dirs, plain_models, tmp_path):
    """python -m cretif_b200 <model> <prompt ids> <max_tokens>, and --dump-logits."""
    cfg, w = plain_models["A"]
    env = dict(os.environ, PYTHONPATH=ROOT)
    run = lambda *a: subprocess.run([sys.executable, "-m", "cretif_b200", model_dirs["A"], *a],
                                    capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    proc = run("5,17,3,9", "6", "--dtype", "float32")
    assert proc.returncode == 0, proc.stderr[-2000:]
    want = pl.greedy(cfg, w, [5, 17, 3, 9], 6, stop_ids={7})
    assert f"generated ids: {want}" in proc.stdout and "tok/s" in proc.stdout
    dump = tmp_path / "top.json"
    proc = run("5 17 3 9", "--dump-logits", str(dump), "--dtype", "float32")
    assert proc.returncode == 0, proc.stderr[-2000:]
    doc = json.loads(dump.read_text())
    logits = pl.forward(cfg, w, [5, 17, 3, 9])[-1]
    assert doc["num_input_tokens"] == 4 and doc["logits_position"] == 3 and doc["top_k"] == 20
    assert doc["top_logits"][0]["token_id"] == int(torch.argmax(logits))
    assert abs(doc["top_logits"][0]["logit_value"] - float(logits.max())) < 1e-4
    bad = run("hello there")
    assert bad.returncode != 0 and "token ids" in (bad.stderr + bad.stdout)


def test_decoding_across_a_context_bucket(engines, plain_models):
    """A decode step is planned for a context bucket (512, 1024, ...), which is part of a
    captured graph's key.  Generation and single-token steps that cross 512 keep giving the
    plain model's tokens and logits on both sides of the boundary, captured or not."""
    eng = engines("C", "float32")
    cfg, w = plain_models["C"]
    assert [eng.context_bucket(n) for n in (1, 512, 513, 1024, 5000)] == [512, 512, 1024, 1024, 1024]
    prompts = [tiny.tokens("C", 505, 5), tiny.tokens("C", 498, 6), tiny.tokens("C", 20, 7)]
    got = eng.generate(prompts, max_tokens=14, stop_ids=[])
    for p, r in zip(prompts, got):
        assert r.tokens == pl.greedy(cfg, w, p, 14)
    runner = eng._backends[(0.0, 0, True)].runner
    assert {key[1] for key in runner.graphs} >= {512, 1024}      # a graph per bucket
    # the step function: the same shape of step before and after the boundary, twice each so
    # that both are captured and replayed
    toks = tiny.tokens("C", 520, 8)
    want = pl.forward(cfg, w, toks).numpy()
    slot = eng.alloc_slot()
    try:
        rows = [eng.step([(slot, toks[:506])], "all").cpu().numpy()]
        for i in range(506, 520):
            rows.append(eng.step([(slot, [toks[i]])], "all").cpu().numpy())
    finally:
        eng.free_slot(slot)
    assert rel_err(np.concatenate(rows), want) <= TOL["float32"]
    assert {k[2] for k in eng._graphs if k[0] == (1,)} >= {512, 1024}


def test_seeds_share_one_set_of_decode_graphs(engines):
    """The sampling kernel reads its seed from device memory, so an engine keeps one backend
    (and its graphs) per temperature and top-k, whatever seeds its callers use, and at most
    four of them."""
    from cretif_b200.engine.generate import MAX_BACKENDS
    eng = engines("A", "float32")
    prompts = [tiny.tokens("A", n, 90 + n) for n in (4, 11)]
    outs = {}
    for seed in (1, 2, 3, 1):
        res = eng.generate(prompts, max_tokens=8, temperature=1.3, top_k=50, seed=seed, stop_ids=[])
        toks = [r.tokens for r in res]
        if seed in outs:
            assert toks == outs[seed]                  # the same seed, the same draws
        outs[seed] = toks
    assert len({str(v) for v in outs.values()}) == 3   # other seeds, other draws
    assert sum(1 for k in eng._backends if k[:2] == (1.3, 50)) == 1
    for t in (0.5, 0.6, 0.7, 0.8, 0.9, 1.0):
        eng.generate(prompts, max_tokens=2, temperature=t, stop_ids=[])
    assert len(eng._backends) <= MAX_BACKENDS
