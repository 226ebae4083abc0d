"""The generation loop's decisions, with a scripted backend on the CPU."""
import pytest

from cretif_b200.engine.generate import GenerationLoop


class ScriptedBackend:
    """Returns tokens from a per-request script and records every call."""

    def __init__(self, scripts):
        self.scripts = scripts            # request index -> list of tokens it will "sample"
        self.log = []
        self.live = {}

    def start_batch(self, request_ids, prompts, reserve_lens):
        assert not self.live
        self.ids = list(request_ids)
        self.cursor = {i: 0 for i in self.ids}
        self.live = {pos: i for pos, i in enumerate(self.ids)}
        self.log.append(("start", tuple(self.ids), tuple(reserve_lens)))

    def _next(self, i):
        tok = self.scripts[i][self.cursor[i]]
        self.cursor[i] += 1
        return tok

    def prefill(self):
        self.log.append(("prefill", tuple(self.ids)))
        return [self._next(i) for i in self.ids]

    def decode(self, active):
        assert all(pos in self.live for pos in active), "a released sequence was stepped"
        self.log.append(("decode", tuple(self.ids[p] for p in active)))
        return [self._next(self.ids[p]) for p in active]

    def release(self, pos):
        assert pos in self.live, "released twice"
        del self.live[pos]
        self.log.append(("release", self.ids[pos]))

    def end_batch(self):
        self.live.clear()
        self.log.append(("end",))


def loop(backend, stop=(9,), capacity=4096, max_len=1024, max_batch=64):
    return GenerationLoop(backend, stop, capacity, max_len, 64, max_batch)


def test_stop_tokens_and_sequences_that_end_earlier():
    be = ScriptedBackend({0: [1, 2, 9, 7, 7], 1: [9], 2: [3, 4, 5, 6, 7, 8]})
    res = loop(be).run([[5, 5], [5], [5, 5, 5]], max_tokens=5)
    assert [r.tokens for r in res] == [[1, 2, 9], [9], [3, 4, 5, 6, 7]]
    assert [r.finish_reason for r in res] == ["stop", "stop", "length"]
    decodes = [e[1] for e in be.log if e[0] == "decode"]
    assert decodes == [(0, 2), (0, 2), (2,), (2,)]        # 1 left after the prefill, 0 later
    assert [e[1] for e in be.log if e[0] == "release"] == [1, 0, 2]
    assert be.log[-1] == ("end",)


def test_max_tokens_counts_the_first_token():
    be = ScriptedBackend({0: [1, 2, 3]})
    res = loop(be).run([[4]], max_tokens=1)
    assert res[0].tokens == [1] and res[0].finish_reason == "length"
    assert not any(e[0] == "decode" for e in be.log)
    res = loop(ScriptedBackend({0: [1]})).run([[4]], max_tokens=0)
    assert res[0].tokens == [] and res[0].finish_reason == "length"


def test_requests_are_cut_into_batches_by_count_and_by_cache_room():
    scripts = {i: [1] * 10 for i in range(5)}
    be = ScriptedBackend(scripts)
    res = loop(be, max_batch=2).run([[1]] * 5, max_tokens=3)
    starts = [e[1] for e in be.log if e[0] == "start"]
    assert starts == [(0, 1), (2, 3), (4,)]
    assert all(r.tokens == [1, 1, 1] for r in res)
    # each request reserves prompt + max_tokens - 1 positions, rounded up to 64
    g = loop(ScriptedBackend(scripts), capacity=256)
    assert g.plan_batches([60, 60, 60, 60, 60], max_tokens=10) == [[0, 1], [2, 3], [4]]
    assert g.plan_batches([10, 10, 10, 10, 10], max_tokens=10) == [[0, 1, 2, 3], [4]]
    be = ScriptedBackend(scripts)
    loop(be, capacity=256).run([[1] * 60] * 3, max_tokens=10)
    assert [e[2] for e in be.log if e[0] == "start"] == [(69, 69), (69,)]


def test_requests_that_cannot_run_are_refused_before_anything_starts():
    be = ScriptedBackend({0: [1]})
    with pytest.raises(ValueError, match="empty"):
        loop(be).run([[]], max_tokens=3)
    with pytest.raises(ValueError, match="longest"):
        loop(be, max_len=8).run([[1] * 9], max_tokens=3)
    with pytest.raises(ValueError, match="cache holds"):
        loop(be, capacity=64, max_len=1024).run([[1] * 100], max_tokens=3)
    assert be.log == []


def test_a_full_context_ends_with_length():
    be = ScriptedBackend({0: [1, 2, 3, 4, 5, 6]})
    res = loop(be, max_len=6).run([[7, 7, 7, 7]], max_tokens=50)
    # positions 0..5: four prompt tokens, then two sampled tokens can be fed back; the third
    # sampled token has no room to be fed, so it is the last
    assert res[0].tokens == [1, 2, 3] and res[0].finish_reason == "length"
    assert [e[2] for e in be.log if e[0] == "start"] == [(6,)]


def test_backend_is_closed_even_when_a_step_fails():
    class Failing(ScriptedBackend):
        def decode(self, active):
            raise RuntimeError("boom")
    be = Failing({0: [1, 2]})
    with pytest.raises(RuntimeError, match="boom"):
        loop(be).run([[1]], max_tokens=4)
    assert be.log[-1] == ("end",)
