"""What the host sees when a kernel reports a fault, without faulting anything: a bounded
wait that runs out, a token id outside the vocabulary in a replayed decode step, and that the
engine goes on correctly afterwards."""
import numpy as np
import pytest
import torch

import plain_llama as pl
import tiny
from replay_cuts import rel_err, run_whole

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_becomes_a_step_error(model_dirs, plain_models):
    from cretif_b200.csrc import ops
    from cretif_b200.engine import Engine, StepError
    eng = Engine(model_dirs["A"], dtype="bfloat16", max_tokens=512)
    cfg, w = plain_models["A"]
    toks = tiny.tokens("A", 40, 3)
    want = pl.forward(cfg, w, toks).numpy()
    assert rel_err(run_whole(eng, toks), want) <= 2e-2
    # one CTA waits 3,000 polls on a barrier nobody completes, gives up and says so
    ops.wait_that_expires(3000, eng.fault)
    with pytest.raises(StepError, match="bounded wait"):
        eng.check_fault()
    assert int(eng.fault.item()) == 0                  # read and cleared
    eng.check_fault()                                  # nothing pending any more
    # a step that meets the bit left by an earlier launch reports it, once
    ops.wait_that_expires(100, eng.fault)
    slot = eng.alloc_slot()
    with pytest.raises(StepError, match="bounded wait"):
        eng.step([(slot, toks)])
    eng.free_slot(slot)
    assert rel_err(run_whole(eng, toks), want) <= 2e-2  # and the engine works as before
    eng.cache.check()
    with pytest.raises(ops.KernelError):
        ops.wait_that_expires(1 << 21, eng.fault)      # the poll limit itself is bounded


@pytest.mark.parametrize("use_graph", [True, False])
def test_a_token_outside_the_vocabulary_in_a_decode_step(model_dirs, plain_models, use_graph):
    """The generation loop's decode step reads its token ids from device memory; an id that
    is out of range there (put there by hand between two steps) sets the status bit in the
    embedding kernel, which writes zeros instead of reading outside the table."""
    from cretif_b200.engine import Engine, StepError
    from cretif_b200.engine.generate import EngineBackend
    from cretif_b200.sampling import SamplingParams
    eng = Engine(model_dirs["B"], dtype="float32", max_tokens=512)
    cfg, w = plain_models["B"]
    prompts = [tiny.tokens("B", n, 40 + n) for n in (5, 12)]
    be = EngineBackend(eng, SamplingParams(), use_graph=use_graph, run_ahead=False)
    be.start_batch([0, 1], prompts, [40, 40])
    try:
        first = be.prefill()
        second = be.decode([0, 1])                     # captured on this call when use_graph
        assert [first[0], second[0]] == pl.greedy(cfg, w, prompts[0], 2)
        be.runner.bufs[2]["tok_ids"][1] = cfg["vocab_size"] + 3
        be.decode([0, 1])
        with pytest.raises(StepError, match="outside the vocabulary"):
            eng.check_fault()
        eng.check_fault()
    finally:
        be.end_batch()
    eng.cache.check()
    assert eng.cache.stats()["slots_live"] == 0
    got = eng.generate(prompts, max_tokens=4, stop_ids=[], use_graph=use_graph)
    for p, r in zip(prompts, got):
        assert r.tokens == pl.greedy(cfg, w, p, 4)
