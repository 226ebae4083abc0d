"""Each part alone against the plain implementation's function for it, and a toy mixer with
state of its own that is registered here, built and stepped without touching the package."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return torch.randn(*shape, generator=g) * scale


def close(got, want, rel):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= rel, f"relative error {err:.3e} > {rel:.1e}"


def make_ctx(cache, slots, starts, news, dtype):
    """A StepContext for sequences in `slots` bringing `news` tokens after `starts` cached."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.base import StepContext
    B, T = len(slots), int(sum(news))
    cu = np.concatenate([[0], np.cumsum(news)])
    tok_seq = np.repeat(np.arange(B), news)
    tok_pos = np.arange(T) - cu[tok_seq] + np.asarray(starts)[tok_seq]
    i32 = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    return StepContext(T=T, B=B, tok_ids=i32(np.zeros(T)), tok_pos=i32(tok_pos), tok_seq=i32(tok_seq),
                       seq_slot=i32(slots), seq_start=i32(starts), cu_seqlens=i32(cu),
                       is_decode=all(n == 1 for n in news), max_new=max(news),
                       max_context=int(max(s + n for s, n in zip(starts, news))),
                       fault=ops.fault_word(DEV), dtype=dtype, device=torch.device(DEV))


# float32: rounding of 32-bit sums.  bfloat16: the suite-wide bound for bfloat16 storage of
# activations and cached keys/values (the same 2e-2 the engine tests use).
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from cretif_b200.parts.base import build_part
    from cretif_b200.config import PartSpec
    H, eps = 88, 2e-5
    part = build_part("norm", PartSpec("rmsnorm", {"eps": eps, "name": "w"}), H, dtype, DEV)
    w = rnd(H) * 0.1 + 1
    part.load({"weight": w.to(torch.bfloat16)})          # stored bf16, applied in 32-bit
    wq = w.to(torch.bfloat16).double()
    h, d = rnd(6, H, seed=1).to(DEV), rnd(6, H, seed=2).to(DEV)
    h2 = h.clone()
    n = part.forward(h2, d)
    assert n.dtype == dtype
    close(h2, h.double() + d.double(), 1e-7)
    close(n, pl.rmsnorm((h.double() + d.double()).cpu(), wq, eps), TOL[dtype])
    n0 = part.forward(h.clone(), None)
    close(n0, pl.rmsnorm(h.double().cpu(), wq, eps), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("window", [0, 50])
def test_attention_part_prefill_then_decode(dtype, pairing, window):
    """The mixer alone, with its position encoding and cache: a ragged prefill of three
    sequences, then decode steps, against the plain functions on whole sequences."""
    from cretif_b200.cache import SequenceCache
    from cretif_b200.config import PartSpec
    from cretif_b200.parts.base import LayerCache, build_part
    H, nh, nkv, hd, theta = 72, 6, 2, 32, 5000.0
    scale = 0.2
    params = {"num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "scale": scale,
              "window": window,
              "position": {"kind": "rotary", "theta": theta, "rotary_dim": hd, "pairing": pairing},
              "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}
    part = build_part("mixer", PartSpec("attention", params), H, dtype, DEV)
    W = {"q": rnd(nh * hd, H, scale=0.2, seed=1), "k": rnd(nkv * hd, H, scale=0.2, seed=2),
         "v": rnd(nkv * hd, H, scale=0.2, seed=3), "o": rnd(H, nh * hd, scale=0.2, seed=4)}
    W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    part.load(W)
    part.prepare(512)
    cache = SequenceCache({0: part.cache_request()}, 1024, dtype, DEV, max_len=512)
    lens, extra = [70, 5, 130], 6
    xs = [rnd(n + extra, H, seed=10 + i).to(torch.bfloat16) for i, n in enumerate(lens)]
    slots = [cache.alloc_slot() for _ in lens]
    rot = pl.rope_interleaved if pairing == "interleaved" else pl.rope_half

    def plain(x):
        x = x.double()
        S = x.shape[0]
        q = (x @ W["q"].double().T).reshape(S, nh, hd)
        k = (x @ W["k"].double().T).reshape(S, nkv, hd)
        v = (x @ W["v"].double().T).reshape(S, nkv, hd)
        q = torch.stack([rot(q[t], t, theta) for t in range(S)])
        k = torch.stack([rot(k[t], t, theta) for t in range(S)])
        o = pl.attention(q, k, v, scale, window=window)
        return o.reshape(S, nh * hd) @ W["o"].double().T
    wants = [plain(x) for x in xs]

    def run(starts, news):
        entries = list(zip(slots, news))
        cache.begin_step(entries)
        ctx = make_ctx(cache, slots, starts, news, dtype)
        x = torch.cat([xs[i][s:s + n] for i, (s, n) in enumerate(zip(starts, news))]).to(DEV).to(dtype)
        y = part.forward(x, ctx, LayerCache(kv=cache.kv_view(0), writes=True))
        cache.end_step(entries)
        return y
    y = run([0, 0, 0], lens)
    assert y.dtype == torch.float32
    o = 0
    for i, n in enumerate(lens):
        close(y[o:o + n], wants[i][:n], TOL[dtype])
        o += n
    rows = [[] for _ in lens]
    for step in range(extra):
        y = run([n + step for n in lens], [1, 1, 1])
        for i in range(len(lens)):
            rows[i].append(y[i])
    for i, n in enumerate(lens):
        close(torch.stack(rows[i]), wants[i][n:n + extra], TOL[dtype])
    cache.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(dtype):
    from cretif_b200.config import PartSpec
    from cretif_b200.parts.base import build_part
    H, I = 72, 200
    part = build_part("feed_forward", PartSpec("gated_mlp", {
        "intermediate_size": I, "activation": "silu",
        "names": {"gate": "g", "up": "u", "down": "d"}}), H, dtype, DEV)
    W = {"gate": rnd(I, H, scale=0.3, seed=1).to(torch.bfloat16),
         "up": rnd(I, H, scale=0.3, seed=2).to(torch.bfloat16),
         "down": rnd(H, I, scale=0.3, seed=3).to(torch.bfloat16)}
    part.load(W)
    for T in (1, 9, 150):                     # decode-sized and prefill-sized
        x = rnd(T, H, seed=T).to(torch.bfloat16)
        y = part.forward(x.to(DEV).to(dtype), None)
        want = pl.swiglu(x.double(), W["gate"].double(), W["up"].double(), W["down"].double())
        close(y, want, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_tied_head(dtype):
    from cretif_b200.config import PartSpec
    from cretif_b200.csrc import ops
    from cretif_b200.parts.base import build_part
    V, H = 333, 40
    emb = build_part("embedding", PartSpec("token_embedding", {"name": "e", "vocab_size": V}), H,
                     dtype, DEV)
    table = rnd(V, H, seed=1).to(torch.bfloat16)
    emb.load({"table": table})
    head = build_part("head", PartSpec("linear_head", {"tied": True, "name": "h",
                                                       "vocab_size": V}), H, dtype, DEV)
    head.load({})
    head.tie(emb)
    assert head.weight.data_ptr() == emb.table.data_ptr() and head.weight_bytes() == 0
    ids = torch.tensor([0, 332, 7], dtype=torch.int32, device=DEV)

    class Ctx:
        fault = ops.fault_word(DEV)
    h = emb.forward(ids, Ctx)
    assert h.dtype == torch.float32
    assert torch.equal(h.cpu(), pl.embed(table.float(), [0, 332, 7]))
    n = rnd(3, H, seed=2).to(torch.bfloat16)
    logits = head.forward(n.to(DEV).to(dtype), Ctx)
    assert logits.dtype == torch.float32 and tuple(logits.shape) == (3, V)
    close(logits, pl.lm_head(n.double(), table.double()), 1e-5 if dtype == torch.float32 else 1e-5)


# ---------------------------------------------------------------------------------------
# A toy architecture defined here: its mixer keeps a running sum of its inputs per sequence
# (fixed-size state, no keys or values) and returns the running mean.
# ---------------------------------------------------------------------------------------
def _register_toy():
    from cretif_b200.cache import StateRequest
    from cretif_b200.config import (ModelSpec, PartSpec, ScheduleEntry, prenorm_layer,
                                    register_architecture)
    from cretif_b200.parts.base import Part, register_part
    from cretif_b200.weights.loader import WeightSpec

    @register_part("mixer", "running_mean")
    class RunningMean(Part):
        """y_t = gain * mean(x_0..x_t); state per sequence: [sum (H floats), count]."""

        @classmethod
        def weight_specs(cls, params, hidden_size):
            return {"gain": (params["name"], WeightSpec((hidden_size,), init=(1.0, 0.1)))}

        def load(self, tensors):
            self.gain = self._vector32(tensors["gain"])

        def cache_request(self):
            return StateRequest((self.hidden_size + 1,), torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            cu = ctx.cu_seqlens.tolist()
            for b, slot in enumerate(ctx.seq_slot.tolist()):
                st = cache.state[slot]
                xs = x[cu[b]:cu[b + 1]].float()
                sums = st[:-1] + torch.cumsum(xs, dim=0)
                counts = st[-1] + torch.arange(1, xs.shape[0] + 1, device=x.device)
                out[cu[b]:cu[b + 1]] = self.gain * sums / counts[:, None]
                if cache.writes:
                    st[:-1] = sums[-1]
                    st[-1] = counts[-1]
            return out

    def config_from_dict(raw):
        return dict(raw)

    def build_spec(cfg):
        H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
        norm = lambda name: PartSpec("rmsnorm", {"eps": 1e-5, "name": name})
        layers = [prenorm_layer(f"blocks.{i}.",
                                mixer=PartSpec("running_mean", {"name": "mix.gain"}),
                                feed_forward=PartSpec("gated_mlp", {
                                    "intermediate_size": cfg["ffn"], "activation": "silu",
                                    "names": {"gate": "ff.g", "up": "ff.u", "down": "ff.d"}}),
                                mixer_norm=norm("n1"), feed_forward_norm=norm("n2"))
                  for i in range(L)]
        return ModelSpec(architecture="ToyRunningMean", vocab_size=cfg["vocab_size"],
                         hidden_size=H, embedding=PartSpec("token_embedding", {"name": "emb"}),
                         layers=layers, schedule=[ScheduleEntry(i) for i in range(L)],
                         final_norm=norm("final"),
                         head=PartSpec("linear_head", {"tied": True, "name": "head",
                                                       "tied_to": "emb"}),
                         max_positions=cfg["max_positions"])
    register_architecture("ToyRunningMean", config_from_dict, build_spec)


def _toy_plain(w, L, ids):
    """The toy model on a whole sequence, in float64."""
    h = pl.embed(w["emb"], ids)
    for i in range(L):
        p = f"blocks.{i}."
        n = pl.rmsnorm(h, w[p + "n1"], 1e-5)
        mean = torch.cumsum(n, dim=0) / torch.arange(1, len(ids) + 1, dtype=torch.float64)[:, None]
        h = h + w[p + "mix.gain"] * mean
        n = pl.rmsnorm(h, w[p + "n2"], 1e-5)
        h = h + pl.swiglu(n, w[p + "ff.g"], w[p + "ff.u"], w[p + "ff.d"])
    return pl.lm_head(pl.rmsnorm(h, w["final"], 1e-5), w["emb"])


def test_a_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    import json
    from replay_cuts import rel_err, run_batch, run_tail_by_one, run_whole
    from cretif_b200.engine import Engine
    from cretif_b200.weights.random_model import write_random_model
    _register_toy()
    cfg = {"architectures": ["ToyRunningMean"], "hidden_size": 48, "num_hidden_layers": 2,
           "ffn": 80, "vocab_size": 120, "max_positions": 256}
    d = str(tmp_path / "toy")
    write_random_model(d, cfg, seed=4, dtype=torch.float32)
    eng = Engine(d, dtype="float32", max_tokens=1024)
    st = eng.cache.stats()
    assert st["groups"] == [] and st["state_bytes"] == eng.cache.max_slots * 2 * 49 * 4
    _, w = pl.read_model_folder(d)
    rng = np.random.default_rng(0)
    reqs = [rng.integers(0, 120, size=n).tolist() for n in (40, 7, 23)]
    wants = [_toy_plain(w, 2, r).numpy() for r in reqs]
    from replay_cuts import run_chunks, run_schedule
    for r, want in zip(reqs, wants):
        assert rel_err(run_whole(eng, r), want) < 1e-4
        assert rel_err(run_tail_by_one(eng, r, tail=10), want) < 1e-4
    # chunks at a cached position: the state carries the scan over
    assert rel_err(run_chunks(eng, reqs[0], [15, 1, 20]), wants[0]) < 1e-4
    outs = run_schedule(eng, reqs, [[(0, 20)], [(0, 13), (1, 7)], [(0, 7), (2, 23)]])
    for got, want in zip(outs, wants):
        assert rel_err(got, want) < 1e-4
    for _ in range(2):          # the second pass takes the slots (and their state) again
        outs = run_batch(eng, reqs, [30, 2, 23])
        for got, want in zip(outs, wants):
            assert rel_err(got, want) < 1e-4
    eng.cache.check()


# ---------------------------------------------------------------------------------------
# A second toy architecture: the library's attention with a position encoding defined here
# (queries and keys are scaled channel by channel with a wave of the position) and a
# feed-forward with routing defined here (the best of three small experts for each token,
# router logits in 32-bit).  Neither becomes part of the framework.
# ---------------------------------------------------------------------------------------
def _wave(pos, hd, amp, freq, dtype=torch.float64):
    """[len(pos), hd] factors 1 + amp · cos(pos · (j + 1) · freq)."""
    j = torch.arange(1, hd + 1, dtype=torch.float64)
    p = torch.as_tensor(pos, dtype=torch.float64)
    return (1.0 + amp * torch.cos(p[:, None] * j[None, :] * freq)).to(dtype)


def _register_routed_toy():
    from cretif_b200.config import (ModelSpec, PartSpec, ScheduleEntry, prenorm_layer,
                                    register_architecture)
    from cretif_b200.csrc import ops
    from cretif_b200.parts.base import Part, register_part
    from cretif_b200.weights.loader import WeightSpec

    @register_part("position", "wave")
    class Wave(Part):
        """q and k of every head are multiplied by _wave(position); nothing is rotated."""

        def load(self, tensors):
            self.amp, self.freq = float(self.params["amp"]), float(self.params["freq"])

        def encode(self, qkv, ctx, nh, nkv, hd):
            w = _wave(ctx.tok_pos.cpu(), hd, self.amp, self.freq).to(qkv.device)
            qk = qkv[:, :(nh + nkv) * hd].unflatten(1, (nh + nkv, hd))
            qk.copy_((qk.double() * w[:, None, :]).to(qkv.dtype))    # the mixer stores them

    @register_part("feed_forward", "best_expert")
    class BestExpert(Part):
        """y = W2[e] · relu(W1[e] · x) for e = argmax(router · x), the router in float32."""

        @classmethod
        def weight_specs(cls, params, hidden_size):
            E, F = params["experts"], params["expert_size"]
            return {"router": ("router", WeightSpec((E, hidden_size), init=(0.0, 1.0))),
                    "w1": ("w1", WeightSpec((E, F, hidden_size))),
                    "w2": ("w2", WeightSpec((E, hidden_size, F)))}

        def load(self, tensors):
            self.router = tensors["router"].to(self.device, torch.float32)
            self.w1 = tensors["w1"].to(self.device, torch.float32)
            self.w2 = tensors["w2"].to(self.device, torch.float32)

        def forward(self, x, ctx):
            x = x.float()
            best = (x @ self.router.T).argmax(dim=-1)                       # [T]
            hidden = torch.relu(torch.einsum("efh,th->tef", self.w1, x))    # every expert
            ys = torch.einsum("ehf,tef->teh", self.w2, hidden)
            return ys[torch.arange(x.shape[0], device=x.device), best]

    def build_spec(cfg):
        H, L, hd = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["head_dim"]
        norm = lambda name: PartSpec("rmsnorm", {"eps": 1e-6, "name": name})
        layers = [prenorm_layer(
            f"l{i}.",
            mixer=PartSpec("attention", {
                "num_heads": cfg["heads"], "num_kv_heads": cfg["kv_heads"], "head_dim": hd,
                "scale": hd ** -0.5, "window": 0,
                "position": {"kind": "wave", "amp": cfg["amp"], "freq": cfg["freq"]},
                "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}),
            feed_forward=PartSpec("best_expert", {"experts": cfg["experts"],
                                                  "expert_size": cfg["expert_size"]}),
            mixer_norm=norm("n1"), feed_forward_norm=norm("n2")) for i in range(L)]
        return ModelSpec(architecture="ToyRouted", vocab_size=cfg["vocab_size"], hidden_size=H,
                         embedding=PartSpec("token_embedding", {"name": "emb"}),
                         layers=layers, schedule=[ScheduleEntry(i) for i in range(L)],
                         final_norm=norm("final"),
                         head=PartSpec("linear_head", {"tied": False, "name": "head",
                                                       "tied_to": "emb"}),
                         max_positions=cfg["max_positions"])
    register_architecture("ToyRouted", lambda raw: dict(raw), build_spec)


def _routed_toy_plain(cfg, w, ids):
    """The second toy model on a whole sequence, in float64; also the router's margins."""
    nh, nkv, hd, L = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    S = len(ids)
    wave = _wave(list(range(S)), hd, cfg["amp"], cfg["freq"])
    h = pl.embed(w["emb"], ids)
    margin = math.inf
    for i in range(L):
        p = f"l{i}."
        n = pl.rmsnorm(h, w[p + "n1"], 1e-6)
        q = (n @ w[p + "q"].T).reshape(S, nh, hd) * wave[:, None, :]
        k = (n @ w[p + "k"].T).reshape(S, nkv, hd) * wave[:, None, :]
        v = (n @ w[p + "v"].T).reshape(S, nkv, hd)
        h = h + pl.attention(q, k, v, hd ** -0.5).reshape(S, nh * hd) @ w[p + "o"].T
        n = pl.rmsnorm(h, w[p + "n2"], 1e-6)
        logits = n @ w[p + "router"].T
        top2 = logits.topk(2, dim=-1).values
        margin = min(margin, float((top2[:, 0] - top2[:, 1]).min()))
        best = logits.argmax(dim=-1)
        y = torch.stack([w[p + "w2"][e] @ torch.relu(w[p + "w1"][e] @ n[t])
                         for t, e in enumerate(best.tolist())])
        h = h + y
    return pl.lm_head(pl.rmsnorm(h, w["final"], 1e-6), w["head"]), margin


def test_a_toy_position_encoding_and_a_routed_feed_forward(tmp_path):
    from replay_cuts import rel_err, run_batch, run_tail_by_one, run_whole
    from cretif_b200.engine import Engine
    from cretif_b200.weights.random_model import write_random_model
    _register_routed_toy()
    cfg = {"architectures": ["ToyRouted"], "hidden_size": 40, "num_hidden_layers": 2,
           "heads": 3, "kv_heads": 1, "head_dim": 16, "experts": 3, "expert_size": 24,
           "amp": 0.4, "freq": 0.37, "vocab_size": 90, "max_positions": 256}
    from cretif_b200.weights import write_model_folder
    d0, d = str(tmp_path / "routed_flat"), str(tmp_path / "routed")
    write_random_model(d0, cfg, seed=11, dtype=torch.float32)
    # Small random weights give nearly uniform attention, which would hide a wrong position
    # factor: queries and keys are scaled up so that each query reads a few particular keys.
    _, w = pl.read_model_folder(d0)
    tensors = {k: v.to(torch.float32) for k, v in w.items()}
    for i in range(cfg["num_hidden_layers"]):
        for name in ("q", "k"):
            tensors[f"l{i}.{name}"] = tensors[f"l{i}.{name}"] * 30.0
    write_model_folder(d, cfg, tensors)
    eng = Engine(d, dtype="float32", max_tokens=1024)
    assert not eng.model.graph_safe          # parts from outside run eagerly unless they say otherwise
    _, w = pl.read_model_folder(d)
    rng = np.random.default_rng(5)
    reqs = [rng.integers(0, 90, size=n).tolist() for n in (70, 9, 33)]
    plain = [_routed_toy_plain(cfg, w, r) for r in reqs]
    # a routing decision on a knife's edge could go either way in 32-bit: there is none here
    assert min(m for _, m in plain) > 1e-3
    wants = [o.numpy() for o, _ in plain]
    for r, want in zip(reqs, wants):
        assert rel_err(run_whole(eng, r), want) < 1e-4
        assert rel_err(run_tail_by_one(eng, r, tail=12), want) < 1e-4
    for _ in range(2):
        for got, want in zip(run_batch(eng, reqs, [50, 3, 33]), wants):
            assert rel_err(got, want) < 1e-4
    eng.cache.check()
    # the position encoding matters: without the wave the logits are others
    flat = dict(cfg, amp=0.0)
    other, _ = _routed_toy_plain(flat, w, reqs[0])
    assert rel_err(other.numpy(), wants[0]) > 1e-2


# ---------------------------------------------------------------------------------------
# A third toy architecture, made of the library's own parts in another block layout: layers
# of ONE branch each.  Even layers are attention behind a norm and nothing else (no
# feed-forward); odd layers are a feed-forward that reads the residual stream as it is and
# whose output is normed AFTER the part, before it is added.  Only a spec builder is
# registered: the engine, the loader, the cache and the random-weights mode follow from it.
# ---------------------------------------------------------------------------------------
def _register_lean_toy():
    from cretif_b200.config import (BranchSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                                    register_architecture)

    def build_spec(cfg):
        H, L, hd = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["head_dim"]
        norm = lambda name: PartSpec("rmsnorm", {"eps": 1e-5, "name": name})
        attn = PartSpec("attention", {
            "num_heads": cfg["heads"], "num_kv_heads": cfg["kv_heads"], "head_dim": hd,
            "scale": hd ** -0.5, "window": 0,
            "position": {"kind": "rotary", "theta": 10000.0, "rotary_dim": hd, "pairing": "half"},
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})
        ffn = PartSpec("gated_mlp", {"intermediate_size": cfg["ffn"], "activation": "silu",
                                     "names": {"gate": "g", "up": "u", "down": "d"}})
        layers = [LayerSpec(f"l{i}.", (BranchSpec("mixer", attn, norm=norm("pre")),))
                  if i % 2 == 0 else
                  LayerSpec(f"l{i}.", (BranchSpec("feed_forward", ffn, post_norm=norm("post")),))
                  for i in range(L)]
        return ModelSpec(architecture="ToyLean", vocab_size=cfg["vocab_size"], hidden_size=H,
                         embedding=PartSpec("token_embedding", {"name": "emb"}),
                         layers=layers, schedule=[ScheduleEntry(i) for i in range(L)],
                         final_norm=norm("final"),
                         head=PartSpec("linear_head", {"tied": True, "name": "head",
                                                       "tied_to": "emb"}),
                         max_positions=cfg["max_positions"])
    register_architecture("ToyLean", lambda raw: dict(raw), build_spec)


def _lean_toy_plain(cfg, w, ids):
    nh, nkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    S = len(ids)
    h = pl.embed(w["emb"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"l{i}."
        if i % 2 == 0:
            n = pl.rmsnorm(h, w[p + "pre"], 1e-5)
            q = (n @ w[p + "q"].T).reshape(S, nh, hd)
            k = (n @ w[p + "k"].T).reshape(S, nkv, hd)
            v = (n @ w[p + "v"].T).reshape(S, nkv, hd)
            q = torch.stack([pl.rope_half(q[t], t, 10000.0) for t in range(S)])
            k = torch.stack([pl.rope_half(k[t], t, 10000.0) for t in range(S)])
            h = h + pl.attention(q, k, v, hd ** -0.5).reshape(S, nh * hd) @ w[p + "o"].T
        else:
            y = pl.swiglu(h, w[p + "g"], w[p + "u"], w[p + "d"])
            h = h + pl.rmsnorm(y, w[p + "post"], 1e-5)
    return pl.lm_head(pl.rmsnorm(h, w["final"], 1e-5), w["emb"])


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 2e-2)])
def test_blocks_of_one_branch_and_a_norm_after_the_part(tmp_path, dtype, tol):
    from replay_cuts import rel_err, run_batch, run_chunks, run_tail_by_one, run_whole
    from cretif_b200.engine import Engine
    from cretif_b200.weights.random_model import write_random_model
    _register_lean_toy()
    cfg = {"architectures": ["ToyLean"], "hidden_size": 64, "num_hidden_layers": 4, "heads": 4,
           "kv_heads": 2, "head_dim": 16, "ffn": 96, "vocab_size": 150, "max_positions": 256}
    d = str(tmp_path / "lean")
    write_random_model(d, cfg, seed=8)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    assert [len(layer.branches) for layer in eng.model.layers] == [1, 1, 1, 1]
    # two of the four layers keep keys and values; the others keep nothing
    assert eng.cache.stats()["groups"][0]["layers"] == 2
    _, w = pl.read_model_folder(d)
    rng = np.random.default_rng(2)
    reqs = [rng.integers(0, 150, size=n).tolist() for n in (70, 9, 33)]
    wants = [_lean_toy_plain(cfg, w, r).numpy() for r in reqs]
    for r, want in zip(reqs, wants):
        assert rel_err(run_whole(eng, r), want) <= tol
        assert rel_err(run_tail_by_one(eng, r, tail=12), want) <= tol
    assert rel_err(run_chunks(eng, reqs[0], [30, 1, 25]), wants[0]) <= tol
    for _ in range(2):
        for got, want in zip(run_batch(eng, reqs, [50, 3, 33]), wants):
            assert rel_err(got, want) <= tol
    eng.cache.check()
