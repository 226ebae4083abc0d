"""A plain, slow Llama: whole sequences, no cache, one function per part.

This is the yardstick the engine is compared with.  It shares no code with the
package: it reads config.json with ``json`` and the weights with the
``safetensors`` library, and computes in float64 (or float32) with elementary
torch arithmetic on the CPU.

It follows the reference's formulas, cited function by function as
``file:line`` within the reference project.  The reference's own model code is
CUDA-only (it has no CPU forward pass that could be imported or compiled on a
machine without a GPU), so it was run once on a GPU instead: the logits its
unmodified program printed for seeded random models lie under ``tests/golden/``
with the script that made them, and ``tests/test_reference_golden.py`` checks on
the CPU that :func:`forward` reproduces them.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def read_model_folder(model_dir: str):
    """config.json as a dict and every tensor of model.safetensors in float64."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(torch.float64)
    return cfg, weights


def embed(table: torch.Tensor, ids: List[int]) -> torch.Tensor:
    """h[t, :] = E[id_t, :], no scaling (src/embedding.cu:39-60)."""
    return torch.stack([table[i] for i in ids])


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x · w · rsqrt(mean(x²) + eps), per row (src/kernels/elementwise.cu:30-72)."""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * weight * (1.0 / torch.sqrt(mean_sq + eps))


def rope_angles(position: int, head_dim: int, theta: float, dtype) -> torch.Tensor:
    """a_j = position / theta^(2j / head_dim), j < head_dim/2
    (src/kernels/elementwise.cu:244-247)."""
    j = torch.arange(head_dim // 2, dtype=torch.float64)
    freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * j / head_dim)
    return (position * freq).to(dtype)


def rope_interleaved(x: torch.Tensor, position: int, theta: float) -> torch.Tensor:
    """Rotate pairs (2j, 2j+1) of each head of x [heads, head_dim] by a_j
    (src/kernels/elementwise.cu:232-258)."""
    hd = x.shape[-1]
    a = rope_angles(position, hd, theta, x.dtype)
    cos, sin = torch.cos(a), torch.sin(a)
    out = torch.empty_like(x)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out[..., 0::2] = x0 * cos - x1 * sin
    out[..., 1::2] = x0 * sin + x1 * cos
    return out


def rope_half(x: torch.Tensor, position: int, theta: float) -> torch.Tensor:
    """The same rotation on pairs (j, j + head_dim/2).

    Llama weight files in the reference's format carry query/key rows permuted
    per head so that its interleaved rotation (src/kernels/elementwise.cu:232-258)
    on them equals this half-split rotation on the unpermuted rows of a
    config.json + safetensors checkpoint; ``test_plain_llama.py`` proves the
    equivalence with :func:`permute_rows_for_interleaved`.
    """
    hd = x.shape[-1]
    a = rope_angles(position, hd, theta, x.dtype)
    cos, sin = torch.cos(a), torch.sin(a)
    x0, x1 = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def permute_rows_for_interleaved(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Rows of a q/k projection [heads·hd, H] reordered so that row 2j+c of a
    head is the unpermuted row c·hd/2 + j."""
    hd = w.shape[0] // n_heads
    w = w.reshape(n_heads, 2, hd // 2, -1)            # [head, c, j, :]
    return w.transpose(1, 2).reshape(n_heads * hd, -1)  # [head, j, c, :]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              start: int = 0, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [S, nh, hd] are the queries at positions start..start+S-1, k/v [start+S, nkv, hd]
    all keys.  Query head h reads key/value head h // (nh/nkv) (src/attention.cu:206-207,
    421-422); s = (q·k)·scale with the scale applied after the dot (:690-692); keys u > p
    are masked (:60-77); softmax with max subtraction (src/kernels/elementwise.cu:154-202);
    o = Σ p·v (src/attention.cu:710-714).  ``window`` W > 0 also masks u ≤ p − W.
    """
    S, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.zeros(S, nh, hd, dtype=q.dtype)
    p = start + torch.arange(S)[:, None]                  # each query's position
    u = torch.arange(k.shape[0])[None, :]                 # each key's position
    hidden = u > p                                        # the causal mask
    if window > 0:
        hidden = hidden | (u <= p - window)
    for h in range(nh):
        kvh = h // g
        scores = (q[:, h, :] @ k[:, kvh, :].T) * scale            # [S, start+S]
        scores = scores.masked_fill(hidden, -math.inf)
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        probs = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = probs @ v[:, kvh, :]
    return out


def swiglu(x: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    """down(silu(gate(x)) ⊙ up(x)), silu(z) = z / (1 + exp(−z)), no bias
    (src/ffn.cu:152-190; src/kernels/elementwise.cu:93-99)."""
    gate = x @ w_gate.T
    up = x @ w_up.T
    act = gate / (1.0 + torch.exp(-gate)) * up
    return act @ w_down.T


def lm_head(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """logits = x · Wᵀ with W [vocab, hidden] (src/embedding.cu:85-135)."""
    return x @ w.T


def forward(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int],
            dtype=torch.float64, rope: Optional[str] = None, storage=None) -> torch.Tensor:
    """Logits [S, vocab] of one whole sequence, layer order of src/model.cu:859-1039:
    embed → per layer {norm → q,k,v → rope(q,k) → attention → o → residual →
    norm → SwiGLU → residual} → final norm → head (tied: the embedding matrix).

    ``storage`` (e.g. ``torch.bfloat16``) rounds the activations that an engine with that
    storage type writes to memory between kernels — normed rows, q/k/v before and after
    the rotation, the attention output, gate/up and their activation — and nothing else:
    sums, softmax, the residual stream and the logits stay in ``dtype``.  It models where a
    reduced-precision engine loses bits, so that inputs with large scores can be compared
    tightly; the reference itself keeps everything in 32-bit (docs/architecture.md:748-753).
    """
    def st(x):
        return x if storage is None else x.to(storage).to(dtype)
    W = {k: v.to(dtype) for k, v in weights.items()}
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    H = cfg["hidden_size"]
    hd = cfg.get("head_dim") or H // nh                      # src/model.cu:541
    eps = cfg.get("rms_norm_eps", 1e-5)                     # src/gguf_parser.cpp:730-736
    theta = cfg.get("rope_theta", 10000.0)                  # src/gguf_parser.cpp:722-728
    if rope is None:
        rope = "interleaved" if cfg.get("rope_interleaved") else "half"
    rot = rope_interleaved if rope == "interleaved" else rope_half
    S = len(ids)
    pos = torch.arange(S, dtype=torch.float64)[:, None]

    def rot_all(x):        # every token's heads rotated by its own position's angles
        if S <= 64:
            return torch.stack([rot(x[t], t, theta) for t in range(S)])
        j = torch.arange(hd // 2, dtype=torch.float64)
        a = (pos / torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * j / hd)).to(dtype)
        cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]      # [S, 1, hd/2]
        if rope == "interleaved":
            x0, x1 = x[..., 0::2], x[..., 1::2]
            return torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1).flatten(-2)
        x0, x1 = x[..., : hd // 2], x[..., hd // 2:]
        return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)

    def window_of(i):      # keys a query of layer i sees (0: all), see config/llama.py
        w = cfg.get("sliding_window")
        kinds = cfg.get("layer_types")
        if w is None or (kinds is not None and kinds[i] != "sliding_attention"):
            return 0
        return int(w)
    h = embed(W["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        n = st(rmsnorm(h, W[p + "input_layernorm.weight"], eps))
        q = st(n @ W[p + "self_attn.q_proj.weight"].T).reshape(S, nh, hd)  # src/attention.cu:567-576
        k = st(n @ W[p + "self_attn.k_proj.weight"].T).reshape(S, nkv, hd)
        v = st(n @ W[p + "self_attn.v_proj.weight"].T).reshape(S, nkv, hd)
        q = st(rot_all(q))                                               # src/attention.cu:589-597
        k = st(rot_all(k))
        o = st(attention(q, k, v, 1.0 / math.sqrt(hd), window=window_of(i)))
        h = h + o.reshape(S, nh * hd) @ W[p + "self_attn.o_proj.weight"].T  # src/attention.cu:720-728
        n = st(rmsnorm(h, W[p + "post_attention_layernorm.weight"], eps))
        if storage is None:
            h = h + swiglu(n, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                           W[p + "mlp.down_proj.weight"])
        else:                                   # the same formula with its stores rounded
            gate = st(n @ W[p + "mlp.gate_proj.weight"].T)
            up = st(n @ W[p + "mlp.up_proj.weight"].T)
            act = st(gate / (1.0 + torch.exp(-gate)) * up)
            h = h + act @ W[p + "mlp.down_proj.weight"].T
    n = st(rmsnorm(h, W["model.norm.weight"], eps))
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else W["lm_head.weight"]
    return lm_head(n, head)


def greedy(cfg: dict, weights, prompt: List[int], max_new_tokens: int,
           stop_ids=(), dtype=torch.float64) -> List[int]:
    """Greedy continuation by re-running the whole sequence each time; ties go to the
    lowest id (src/embedding.cu:155-204).  A sampled stop id ends the sequence and is
    kept (src/model.cu:1081-1095)."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(max_new_tokens):
        logits = forward(cfg, weights, ids, dtype)[-1]
        best = int(torch.nonzero(logits == logits.max())[0])
        out.append(best)
        ids.append(best)
        if best in stop_ids:
            break
    return out
