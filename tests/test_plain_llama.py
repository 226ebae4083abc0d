"""The plain implementation itself: its parts against hand-made cases."""
import math

import pytest
import torch

import plain_llama as pl
import tiny


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    out = pl.rmsnorm(x, w, 0.0)
    r = 1.0 / math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[6.0 * r, 2.0 * r]], dtype=torch.float64))


def test_rope_is_a_rotation_and_identity_at_zero():
    x = torch.randn(3, 16, dtype=torch.float64)
    for rot in (pl.rope_interleaved, pl.rope_half):
        assert torch.allclose(rot(x, 0, 10000.0), x)
        y = rot(x, 17, 10000.0)
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # first pair turns by `position` radians (frequency 1)
    e = torch.zeros(1, 8, dtype=torch.float64)
    e[0, 0] = 1.0
    y = pl.rope_interleaved(e, 2, 10000.0)
    assert torch.allclose(y[0, :2], torch.tensor([math.cos(2.0), math.sin(2.0)], dtype=torch.float64))
    y = pl.rope_half(e, 2, 10000.0)
    assert abs(y[0, 0] - math.cos(2.0)) < 1e-12 and abs(y[0, 4] - math.sin(2.0)) < 1e-12


def test_half_rotation_equals_interleaved_rotation_on_permuted_rows():
    """Scores q·k are the same whether unpermuted rows are rotated in halves or permuted
    rows are rotated in interleaved pairs: the two weight layouts give one function."""
    torch.manual_seed(0)
    nh, hd, H = 3, 16, 20
    wq, wk = torch.randn(nh * hd, H, dtype=torch.float64), torch.randn(nh * hd, H, dtype=torch.float64)
    x = torch.randn(5, H, dtype=torch.float64)
    q, k = (x @ wq.T).reshape(5, nh, hd), (x @ wk.T).reshape(5, nh, hd)
    qp = (x @ pl.permute_rows_for_interleaved(wq, nh).T).reshape(5, nh, hd)
    kp = (x @ pl.permute_rows_for_interleaved(wk, nh).T).reshape(5, nh, hd)
    for i in range(5):
        for j in range(5):
            a = (pl.rope_half(q[i], i, 1e4) * pl.rope_half(k[j], j, 1e4)).sum(-1)
            b = (pl.rope_interleaved(qp[i], i, 1e4) * pl.rope_interleaved(kp[j], j, 1e4)).sum(-1)
            assert torch.allclose(a, b)


def test_whole_model_is_the_same_function_in_both_layouts(plain_models):
    cfg, w = plain_models["A"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    wp = dict(w)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}.self_attn."
        wp[p + "q_proj.weight"] = pl.permute_rows_for_interleaved(w[p + "q_proj.weight"], nh)
        wp[p + "k_proj.weight"] = pl.permute_rows_for_interleaved(w[p + "k_proj.weight"], nkv)
    ids = tiny.tokens("A", 11, 3)
    a = pl.forward(cfg, w, ids, rope="half")
    b = pl.forward(cfg, wp, ids, rope="interleaved")
    assert torch.allclose(a, b, atol=1e-12)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(1)
    S, nh, nkv, hd = 6, 4, 2, 8
    q, k, v = (torch.randn(S, n, hd, dtype=torch.float64) for n in (nh, nkv, nkv))
    out = pl.attention(q, k, v, 0.5)
    # the first token sees only itself
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])
    # a later key does not change an earlier output
    k2, v2 = k.clone(), v.clone()
    k2[5] += 10.0
    v2[5] -= 3.0
    out2 = pl.attention(q, k2, v2, 0.5)
    assert torch.allclose(out[:5], out2[:5]) and not torch.allclose(out[5], out2[5])
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v3 = v.clone()
    v3[:, 1] += 1.0
    out3 = pl.attention(q, k, v3, 0.5)
    assert torch.allclose(out[:, :2], out3[:, :2]) and torch.allclose(out[:, 2:] + 1.0, out3[:, 2:])
    # window 1: every token sees only itself
    assert torch.allclose(pl.attention(q, k, v, 0.5, window=1)[:, 0], v[:, 0])
    # a continuation (start > 0) equals the tail of the whole
    tail = pl.attention(q[4:], k, v, 0.5, start=4)
    assert torch.allclose(tail, out[4:])


def test_swiglu_and_head_by_hand():
    x = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    wg = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    wu = torch.tensor([[0.0, 1.0]], dtype=torch.float64)
    wd = torch.tensor([[2.0], [3.0]], dtype=torch.float64)
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    out = pl.swiglu(x, wg, wu, wd)
    assert torch.allclose(out, torch.tensor([[2.0 * silu1 * -2.0, 3.0 * silu1 * -2.0]],
                                            dtype=torch.float64))
    wh = torch.tensor([[1.0, 1.0], [0.5, 0.0], [0.0, -1.0]], dtype=torch.float64)
    assert torch.allclose(pl.lm_head(x, wh), torch.tensor([[-1.0, 0.5, 2.0]], dtype=torch.float64))
    assert pl.lm_head(x, torch.randn(7, 2, dtype=torch.float64)).shape == (1, 7)


def test_forward_prefix_property_and_greedy(plain_models):
    """Logits at a position depend only on the tokens up to it."""
    for name in ("A", "B", "C"):
        cfg, w = plain_models[name]
        ids = tiny.tokens(name, 12, 4)
        full = pl.forward(cfg, w, ids)
        part = pl.forward(cfg, w, ids[:7])
        assert full.shape == (12, cfg["vocab_size"])
        assert torch.allclose(full[:7], part, atol=1e-12)
    cfg, w = plain_models["A"]
    out = pl.greedy(cfg, w, [1, 2, 3], 4)
    assert len(out) == 4
    first = int(torch.argmax(pl.forward(cfg, w, [1, 2, 3])[-1]))
    assert out[0] == first
    assert pl.greedy(cfg, w, [1, 2, 3], 4, stop_ids={first}) == [first]


def test_float32_plain_is_close_to_float64(plain_models):
    cfg, w = plain_models["B"]
    ids = tiny.tokens("B", 20, 5)
    a = pl.forward(cfg, w, ids)
    b = pl.forward(cfg, w, ids, dtype=torch.float32)
    assert (a - b.double()).abs().max() / a.abs().max() < 1e-5
