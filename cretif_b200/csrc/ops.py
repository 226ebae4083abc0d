"""Python faces of the CUDA launchers: argument checks, then one ctypes call each.

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, sizes) and raises ``KernelError`` with a plain message when a kernel
refuses its arguments.  There is no fallback of any kind: without the compiled
library, or with a tensor that is not on a CUDA device, the call fails.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_STATUS = {-1: "sizes or options the kernel does not take", -2: "unsupported element type",
           -3: "pointer or row stride not aligned as the kernel needs"}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = load_library()
        L.cretif_uniform01.restype = ctypes.c_float
        L.cretif_uniform01.argtypes = [ctypes.c_ulonglong, ctypes.c_longlong, ctypes.c_int]
        _lib = L
    return _lib


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (graph replays are not counted)."""
    return _launches


_VARIANTS = ("fused_registers", "fused_row_groups", "fused_cluster2", "fused_cluster4", "stream",
             "stream_row_groups", "decode_cluster", "decode_split", "prefill_attn", "tc64",
             "tc128", "tc256", "tc_several_tiles", "tc192", "prefill_attn_pair",
             "prefill_attn_split", "tc_bulk_add", "tc_pair")


def variant_counts() -> dict:
    """How often each variant of the kernels has been launched so far (the order is that of
    ``cretif::Variant``); tests take differences to know which path a step took.  Launches
    replayed from a CUDA graph are not counted."""
    L = lib()
    return {name: int(L.cretif_variant_count(i)) for i, name in enumerate(_VARIANTS)}


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: {_STATUS.get(code, f'status {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"tensors of dtype {t.dtype} have no kernel") from None


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device as a pointer (the raw getter is an order
    of magnitude cheaper than building a torch.cuda.Stream object for every launch)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    try:
        if t.is_cuda and (dtype is None or t.dtype == dtype) and (dim is None or t.dim() == dim):
            return
    except AttributeError:
        pass
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    raise KernelError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


def _rows(t: torch.Tensor, name: str) -> int:
    """Row stride (in elements) of a 2-d tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-d with dense rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0)


# ------------------------------------------------------------------ elementwise
def embed_rows(table, ids, out, fault) -> None:
    _need(table, "table", dim=2); _need(ids, "ids", torch.int32, 1)
    _need(out, "out", torch.float32, 2); _need(fault, "fault", torch.int32)
    T, (V, H) = ids.numel(), table.shape
    if tuple(out.shape) != (T, H) or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError(f"embed_rows: out must be a contiguous [{T}, {H}] tensor")
    _check(lib().cretif_embed_rows(_p(table), _dt(table), _p(ids), _p(out), T, H, V, _p(fault),
                                   _stream()), "embed_rows")


def add_rmsnorm(h, delta, weight, out, eps: float, rows=None, write_h: bool = True) -> None:
    _need(h, "h", torch.float32, 2); _need(weight, "weight", torch.float32, 1)
    _need(out, "out", dim=2)
    H = h.shape[1]
    if not h.is_contiguous() or not out.is_contiguous() or weight.numel() != H:
        raise KernelError("add_rmsnorm: h and out must be contiguous and weight have H elements")
    if delta is not None:
        _need(delta, "delta", dim=2)
        if tuple(delta.shape) != tuple(h.shape) or not delta.is_contiguous():
            raise KernelError("add_rmsnorm: delta must match h")
    R = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        if rows.numel() != R:
            raise KernelError("add_rmsnorm: one source row per output row")
        write_h = False
    elif R != h.shape[0]:
        raise KernelError("add_rmsnorm: out must have as many rows as h")
    if out.shape[1] != H:
        raise KernelError("add_rmsnorm: out has another width than h")
    _check(lib().cretif_add_rmsnorm(_p(h), _p(delta), _dt(delta) if delta is not None else 0,
                                    _p(weight), _p(out), _dt(out), _p(rows), R, H,
                                    ctypes.c_float(eps), int(write_h), _stream()), "add_rmsnorm")


def silu_mul(gu, act, block: int = 0) -> None:
    """act = silu(gate) * up.  ``block`` = 0: gu rows are [gate | up]; ``block`` = b: groups of b
    gate columns each followed by their b up columns."""
    _need(gu, "gu", dim=2); _need(act, "act", gu.dtype, 2)
    T, I = act.shape
    if tuple(gu.shape) != (T, 2 * I) or not gu.is_contiguous() or not act.is_contiguous():
        raise KernelError(f"silu_mul: gu must be contiguous [{T}, {2 * I}]")
    _check(lib().cretif_silu_mul(_p(gu), _p(act), _dt(gu), T, I, block, _stream()), "silu_mul")


def rope_kv_append(qkv, cos, sin, pairing: int, rot_dim: int, nh: int, nkv: int, hd: int,
                   tok_pos, tok_seq=None, seq_slot=None, table=None, kc=None, vc=None,
                   block_tokens: int = 64, write_cache: bool = True, fault=None,
                   rotate_k_in_place: bool = False) -> None:
    """Position-encode q (in place) and k of the packed ``[T, (nh + 2 nkv) hd]`` rows by a
    rotation table, and/or store k and v at each token's position in the block cache.
    ``write_cache``: rotated k, and v, go to the cache; ``rotate_k_in_place``: k is rotated in
    the buffer as well (encoding alone).  ``rot_dim`` 0 rotates nothing (storing alone)."""
    _need(qkv, "qkv", dim=2)
    T, ld = qkv.shape[0], _rows(qkv, "qkv")
    if rot_dim:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if (cos.shape[1] != rot_dim // 2 or not cos.is_contiguous() or not sin.is_contiguous()):
            raise KernelError("rope_kv_append: cos/sin must be contiguous [positions, rot_dim/2]")
    else:
        cos = sin = None                       # nothing is rotated: the tables are not read
    _need(tok_pos, "tok_pos", torch.int32, 1)
    if write_cache:
        for t, n in ((tok_seq, "tok_seq"), (seq_slot, "seq_slot")):
            _need(t, n, torch.int32, 1)
        _need(table, "table", torch.int32, 2)
        _need(kc, "k cache", qkv.dtype, 4); _need(vc, "v cache", qkv.dtype, 4)
        if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
                or not vc.is_contiguous() or kc.shape != vc.shape):
            raise KernelError("rope_kv_append: cache must be contiguous "
                              f"[blocks, {nkv}, {block_tokens}, {hd}], got {tuple(kc.shape)}")
    if fault is None:
        fault = fault_word(qkv.device)
    flags = (1 if write_cache else 0) | (2 if rotate_k_in_place else 0)
    _check(lib().cretif_rope_kv_append(
        _p(qkv), ld, _dt(qkv), _p(cos), _p(sin), pairing, rot_dim, nh, nkv, hd, _p(tok_pos),
        _p(tok_seq), _p(seq_slot), _p(table), table.stride(0) if table is not None else 0,
        _p(kc), _p(vc), block_tokens, flags, T, _p(fault), _stream()), "rope_kv_append")


def advance_decode(tok_ids, tok_pos, seq_start, sampled, B: int) -> None:
    _check(lib().cretif_advance_decode(_p(tok_ids), _p(tok_pos), _p(seq_start), _p(sampled), B,
                                       _stream()), "advance_decode")


# ------------------------------------------------------------------ matrix products
def gemm_simt(a, w, c, accumulate: bool = False) -> None:
    """c[M,N] (+)= a[M,K] · w[N,K]ᵀ in 32-bit FMA arithmetic."""
    _need(a, "a", dim=2); _need(w, "w", dim=2); _need(c, "c", dim=2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(c.shape) != (M, N):
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(c.shape)}")
    _check(lib().cretif_gemm_simt(_p(a), _dt(a), _p(w), _dt(w), _p(c), _dt(c), M, N, K,
                                  _rows(a, "a"), _rows(w, "w"), _rows(c, "c"), int(accumulate),
                                  _stream()), "gemm_simt")


# ------------------------------------------------------------------ attention
def attn_simt(q, out, kc, vc, table, tok_pos, tok_seq, seq_slot, nh: int, nkv: int, hd: int,
              scale: float, window: int, block_tokens: int) -> None:
    _need(q, "q", dim=2); _need(out, "out", q.dtype, 2)
    _need(kc, "k cache", q.dtype, 4); _need(vc, "v cache", q.dtype, 4)
    T = q.shape[0]
    if out.shape[0] != T or out.shape[1] < nh * hd or q.shape[1] < nh * hd:
        raise KernelError("attention: q/out must hold [tokens, heads*head_dim]")
    if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
            or not vc.is_contiguous()):
        raise KernelError("attention: cache must be contiguous [blocks, kv_heads, block, head_dim]")
    if hd % 8 or hd > 256:
        raise KernelError(f"attention: head_dim {hd} is not a multiple of 8 up to 256")
    _check(lib().cretif_attn_simt(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _dt(q), _p(kc), _p(vc), _p(table),
        table.stride(0), _p(tok_pos), _p(tok_seq), _p(seq_slot), nh, nkv, hd,
        ctypes.c_float(scale), window, block_tokens, T, _stream()), "attn_simt")


# ------------------------------------------------------------------ sampling
def sample(logits, out, temperature: float, top_k: int, seed: int, request=None,
           draw=None, seed_dev=None) -> None:
    """``seed_dev`` (one int64 on the device), when given, is read by the kernel instead of
    ``seed``: a captured launch then serves any seed."""
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    rows, V = logits.shape
    if out.numel() < rows:
        raise KernelError("sample: out is shorter than the number of rows")
    if request is not None:
        _need(request, "request", torch.int64, 1)
    if draw is not None:
        _need(draw, "draw", torch.int32, 1)
    if seed_dev is not None:
        _need(seed_dev, "seed_dev", torch.int64, 1)
    if temperature > 0 and 0 < top_k < V and top_k > lib().cretif_max_top_k():
        raise KernelError(f"sample: top_k {top_k} exceeds the kernel's limit "
                          f"{lib().cretif_max_top_k()}")
    _check(lib().cretif_sample(_p(logits), _rows(logits, "logits"), rows, V,
                               ctypes.c_float(temperature), int(top_k),
                               ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _p(seed_dev),
                               _p(request), _p(draw), _p(out), _stream()), "sample")


def uniform01(seed: int, request: int, draw: int) -> float:
    """The uniform number the sampling kernel uses for (seed, request, draw)."""
    return float(lib().cretif_uniform01(ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF),
                                        ctypes.c_longlong(request), draw))


# ------------------------------------------------------------------ fast products (bfloat16)
def gemv_supported(x, w, out) -> bool:
    """The weight-streaming kernel takes bfloat16 operands with 16-byte aligned rows."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= 64
            and K % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and out.dtype in (torch.bfloat16, torch.float32))


def gemv_bf16(x, w, out, accumulate: bool = False) -> None:
    """out[M,N] (+)= x[M,K] · w[N,K]ᵀ for M <= 64 (decode), tensor-core FMA, 32-bit sums."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", dim=2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemv: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _check(lib().cretif_gemm_skinny(_p(x), _p(w), _p(out), _dt(out), M, N, K, _rows(x, "x"),
                                    _rows(w, "w"), _rows(out, "out"), int(accumulate),
                                    _stream()), "gemm_skinny")


_FAULT = {}


def fault_word(device) -> torch.Tensor:
    """The int32 status word of a device that kernels OR their fault bits into."""
    key = str(torch.device(device))
    if key not in _FAULT:
        _FAULT[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _FAULT[key]


def wait_that_expires(limit: int = 2000, fault=None) -> None:
    """Launch one CTA whose bounded wait runs out after ``limit`` polls: it sets the
    "wait expired" bit of the status word and returns.  Harmless; for exercising the path
    from an expired wait to the host's error."""
    if fault is None:
        fault = fault_word(torch.device("cuda", torch.cuda.current_device()))
    _need(fault, "fault", torch.int32)
    _check(lib().cretif_wait_that_expires(int(limit), _p(fault), None, _stream()),
           "wait_that_expires")


def gemm_tc_supported(x, w, out) -> bool:
    """The tensor-core kernel takes bfloat16 operands whose rows are 16-byte aligned."""
    K = x.shape[1]
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0):
        return False
    if out.dtype == torch.bfloat16:
        return out.stride(0) % 8 == 0
    return out.dtype == torch.float32 and out.stride(0) % 4 == 0


def set_tc_epilogue_warps(n: int) -> int:
    """(For tests that run both.)  Epilogue warps of the tensor-core product: 4 or 8; 0 lets
    each launch choose.  Returns the old setting."""
    return int(lib().cretif_set_tc_epilogue_warps(int(n)))


def gemm_tc(x, w, out, accumulate: bool = False, bn: int = 0) -> None:
    """out[M,N] (+)= x[M,K] · w[N,K]ᵀ with TMA, tcgen05.mma and a TMEM accumulator."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", dim=2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _check(lib().cretif_gemm_tc(_p(x), _p(w), _p(out), _dt(out), M, N, K, _rows(x, "x"),
                                _rows(w, "w"), _rows(out, "out"), int(accumulate), bn,
                                _p(fault_word(x.device)), _stream()), "gemm_tc")


# ------------------------------------------------------------------ fast attention (bfloat16)
_SM_COUNT = {}


def sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SM_COUNT[key]


def attn_decode_supported(hd: int, block_tokens: int, group: int = 1) -> bool:
    return block_tokens == 64 and hd % 16 == 0 and 16 <= hd <= 256 and group <= 8


def decode_splits(B: int, nkv: int, max_context: int, device) -> int:
    """Ranges per (sequence, kv head): enough CTAs for about four per SM, at most one per
    cache block of the longest context."""
    tiles = max(1, -(-max_context // 64))
    want = (3 * sm_count(device)) // max(1, B * nkv)      # about three CTAs fit an SM: one wave
    return max(1, min(tiles, want, 64))


CLUSTER_MAX_RANGES = 8


def decode_plan(B: int, nkv: int, max_context: int, device, hd: int = 64):
    """(ranges per (sequence, kv head), merge inside a cluster?) for the decode attention.

    Up to eight ranges can be one thread-block cluster, whose merge through distributed
    shared memory is some 5 us shorter than the one through global scratch; a range is a
    cache block or more, and a block costs about 0.3 us.  So the cluster is taken unless it
    would make a CTA walk 16 blocks more than the plain split would (a long context with
    few sequences).  Cluster sizes are powers of two: at batch 16 and 32 of a 3-kv-head model
    clusters of 6 and 3 took 13.8 and 20.0 us against 9.2 and 12.7 us for 4.  A grid beyond two
    CTAs per SM runs with the shallow ring and in more than one wave, which ranges of up to
    sixteen blocks do not pay for (batch 16 with 8 and 4 ranges: 11.0 and 9.2 us at a context
    of 2,100, 14.3 and 11.5 us at 3,000, 16.4 and 13.7 us at 4,000), so a cluster of 8 becomes
    one of 4 there (4 against 2 at batch 32: 12.7 and 14.3 us, so no further).  (Clusters of
    16, which the hardware takes as an opt-in size, were measured: no gain for one sequence,
    twice the time for eight: too few of them fit the chip at once.)"""
    tiles = max(1, -(-max_context // 64))
    n_split = decode_splits(B, nkv, max_context, device)
    if hd > 128 or _decode_simt_only:
        return n_split, False
    n_cluster = max(1, min(n_split, tiles, CLUSTER_MAX_RANGES))
    n_cluster = 1 << (n_cluster.bit_length() - 1)     # clusters of 3, 6 or 7 CTAs place badly
    if n_cluster > 4 and n_cluster * B * nkv > 2 * sm_count(device) and tiles <= 16 * n_cluster:
        n_cluster //= 2
    if -(-tiles // n_cluster) - -(-tiles // n_split) < 16:
        return n_cluster, True
    return n_split, False


def attn_decode(q, out, kc, vc, table, tok_pos, tok_seq, seq_slot, nh: int, nkv: int, hd: int,
                scale: float, window: int, block_tokens: int, n_splits: int, fault,
                cluster: bool = False) -> None:
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(kc, "k cache", torch.bfloat16, 4); _need(vc, "v cache", torch.bfloat16, 4)
    B = q.shape[0]
    if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
            or not vc.is_contiguous()):
        raise KernelError("attn_decode: cache must be contiguous [blocks, kv_heads, 64, head_dim]")
    if n_splits > 64:
        raise KernelError("attn_decode: at most 64 ranges per (sequence, kv head)")
    if cluster:
        if hd > 128 or _decode_simt_only or n_splits > CLUSTER_MAX_RANGES:
            raise KernelError("attn_decode: the cluster merge takes head sizes up to 128 and at "
                              f"most {CLUSTER_MAX_RANGES} ranges")
        _check(lib().cretif_attn_decode_mma(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(kc), _p(vc),
            ctypes.c_longlong(kc.shape[0]), _p(table), table.stride(0), _p(tok_pos), _p(tok_seq),
            _p(seq_slot), nh, nkv, hd, ctypes.c_float(scale), window, block_tokens, B, n_splits,
            None, None, None, _p(fault), _stream()), "attn_decode_mma")
        return
    part_o = torch.empty((B, nh, n_splits, hd), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((B, nh, n_splits, 2), dtype=torch.float32, device=q.device)
    counters = _decode_counters(q.device, B * nkv)
    if hd <= 128 and not _decode_simt_only:
        _check(lib().cretif_attn_decode_mma(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(kc), _p(vc),
            ctypes.c_longlong(kc.shape[0]), _p(table), table.stride(0), _p(tok_pos), _p(tok_seq),
            _p(seq_slot), nh, nkv, hd, ctypes.c_float(scale), window, block_tokens, B, n_splits,
            _p(part_o), _p(part_ml), _p(counters), _p(fault), _stream()), "attn_decode_mma")
        return
    _check(lib().cretif_attn_decode(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(kc), _p(vc), _p(table),
        table.stride(0), _p(tok_pos), _p(tok_seq), _p(seq_slot), nh, nkv, hd,
        ctypes.c_float(scale), window, block_tokens, B, n_splits, _p(part_o), _p(part_ml),
        _p(counters), _p(fault), _stream()), "attn_decode")


_COUNTERS = {}
_decode_simt_only = False


def decode_attention_simt_only(on: bool) -> None:
    """Use the CUDA-core decode attention kernel even where the tensor-core one applies
    (it is the only one for head sizes above 128; tests run both)."""
    global _decode_simt_only
    _decode_simt_only = bool(on)


def _decode_counters(device, n: int) -> torch.Tensor:
    """Zeroed int32 counters the decode attention uses to find its last CTA; every launch
    leaves them zero, so one buffer per device serves all launches on a stream."""
    key = str(torch.device(device))
    if key not in _COUNTERS or _COUNTERS[key].numel() < n:
        _COUNTERS[key] = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
    return _COUNTERS[key]


# ------------------------------------------------------------------ fused decode projections
FUSED_MAX_ROWS = 128     # the kernels' limit; the parts choose how far they use it
# Beyond 32 rows the kernels read the matrix once per group of 16 or 32 rows: worth it while
# the matrix is small (measured at 64 tokens: 0.7 of the tensor-core path's time at
# SmolLM2-135M sizes, where no matrix but the head exceeds 4 MB, 0.83 at 360M sizes (up to
# 10 MB), 1.2 at 1.7B sizes (25 to 67 MB)).
FUSED_GROUPS_MAX_BYTES = 16 << 20


def fused_supported(M: int, K: int, w, norm: bool = True) -> bool:
    """Whether the fused kernel takes M rows of width K against w (``norm``: with the norm
    prologue, which keeps the normed rows in shared memory)."""
    if M > 32 and w.numel() * w.element_size() > FUSED_GROUPS_MAX_BYTES:
        return False
    return (w.dtype == torch.bfloat16 and 0 < M <= FUSED_MAX_ROWS and K % 8 == 0
            and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and bool(lib().cretif_fused_smem_ok(M, K, int(norm))))


def set_stream_min_k(k: int, min_bytes: int = -1) -> int:
    """(For tests that must run both variants of the fused product on one shape.)  The fused product streams weights through shared memory for matrices of at least k
    columns or (if not negative) at least min_bytes bytes; returns the old column count."""
    return int(lib().cretif_set_stream_min_k(int(k), ctypes.c_longlong(int(min_bytes))))


def stream_min_bytes() -> int:
    """The size threshold of set_stream_min_k."""
    fn = lib().cretif_stream_min_bytes
    fn.restype = ctypes.c_longlong
    return int(fn())


def set_fused_cluster(n: int) -> int:
    """Largest thread-block cluster that shares the norm prologue of the register variant
    (more than eight rows; 1: none, at most 4); returns the old value."""
    return int(lib().cretif_set_fused_cluster(int(n)))


def set_dependent_launch(on: bool) -> bool:
    """Programmatic dependent launch of the fused kernels on or off; returns the old setting."""
    return bool(lib().cretif_set_dependent_launch(int(on)))


def fused_norm_linear(h, norm_w, eps: float, w, out, rows=None, accumulate: bool = False) -> None:
    """out (+)= bf16(rmsnorm(h[rows])) · wᵀ in one kernel (decode-sized row counts)."""
    _need(h, "h", torch.float32, 2); _need(norm_w, "norm weight", torch.float32, 1)
    _need(w, "w", torch.bfloat16, 2); _need(out, "out", dim=2)
    K = h.shape[1]
    M = h.shape[0] if rows is None else rows.numel()
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or not h.is_contiguous():
        raise KernelError("fused_norm_linear: shapes do not fit")
    _check(lib().cretif_fused_linear(None, 0, _p(h), _p(norm_w), _p(rows), ctypes.c_float(eps),
                                     _p(w), _rows(w, "w"), _p(out), _dt(out), _rows(out, "out"),
                                     int(accumulate), M, N, K, _p(fault_word(h.device)),
                                     _stream()), "fused_norm_linear")


def fused_linear_add(x, w, h) -> None:
    """h += x · wᵀ (x bfloat16, h the float32 residual stream)."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2)
    _need(h, "h", torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(h.shape) != (M, N):
        raise KernelError("fused_linear_add: shapes do not fit")
    _check(lib().cretif_fused_linear(_p(x), _rows(x, "x"), None, None, None, ctypes.c_float(0.0),
                                     _p(w), _rows(w, "w"), _p(h), F32, _rows(h, "h"), 1, M, N, K,
                                     _p(fault_word(h.device)), _stream()), "fused_linear_add")


def fused_qkv_rope(h, norm_w, eps: float, w_qkv, q_out, cos, sin, pairing: int, nh: int,
                   nkv: int, hd: int, tok_pos, tok_seq, seq_slot, table, kc, vc,
                   block_tokens: int, write_cache: bool, fault) -> None:
    """norm → q|k|v product → rotary → q buffer and block cache, one kernel."""
    _need(h, "h", torch.float32, 2); _need(w_qkv, "w_qkv", torch.bfloat16, 2)
    _need(q_out, "q", torch.bfloat16, 2)
    M, K = h.shape
    if w_qkv.shape != ((nh + 2 * nkv) * hd, K) or not h.is_contiguous():
        raise KernelError("fused_qkv_rope: shapes do not fit")
    if cos.shape[1] != hd // 2:
        raise KernelError("fused_qkv_rope: needs rotary_dim == head_dim")
    _check(lib().cretif_fused_qkv_rope(
        _p(h), _p(norm_w), ctypes.c_float(eps), _p(w_qkv), _rows(w_qkv, "w_qkv"), _p(q_out),
        _rows(q_out, "q"), _p(cos), _p(sin), pairing, nh, nkv, hd, _p(tok_pos), _p(tok_seq),
        _p(seq_slot), _p(table), table.stride(0), _p(kc), _p(vc), block_tokens,
        int(write_cache), M, K, _p(fault), _stream()), "fused_qkv_rope")


def fused_gate_up_silu(h, norm_w, eps: float, w_gu, act, block: int = 0) -> None:
    """act = silu(norm(h)·Wgᵀ) ⊙ (norm(h)·Wuᵀ), one kernel; w_gu = [Wg; Wu] stacked
    (``block`` = 0) or with rows interleaved in groups of ``block``."""
    _need(h, "h", torch.float32, 2); _need(w_gu, "w_gu", torch.bfloat16, 2)
    _need(act, "act", torch.bfloat16, 2)
    M, K = h.shape
    I = act.shape[1]
    if tuple(w_gu.shape) != (2 * I, K) or act.shape[0] != M or not act.is_contiguous():
        raise KernelError("fused_gate_up_silu: shapes do not fit")
    _check(lib().cretif_fused_gate_up_silu(_p(h), _p(norm_w), ctypes.c_float(eps), _p(w_gu),
                                           _rows(w_gu, "w_gu"), _p(act), I, block, M, K,
                                           _p(fault_word(h.device)), _stream()),
           "fused_gate_up_silu")


def gemm_tc_silu(x, w_gu, act) -> None:
    """act = silu(x·Wgᵀ) ⊙ (x·Wuᵀ) on the tensor cores; w_gu rows interleaved in groups of 64."""
    _need(x, "x", torch.bfloat16, 2); _need(w_gu, "w_gu", torch.bfloat16, 2)
    _need(act, "act", torch.bfloat16, 2)
    M, K = x.shape
    I = act.shape[1]
    if tuple(w_gu.shape) != (2 * I, K) or act.shape[0] != M or not act.is_contiguous():
        raise KernelError("gemm_tc_silu: shapes do not fit")
    _check(lib().cretif_gemm_tc_silu(_p(x), _p(w_gu), _p(act), M, I, K, _rows(x, "x"),
                                     _rows(w_gu, "w_gu"), _p(fault_word(x.device)), _stream()),
           "gemm_tc_silu")


def gemm_tc_qkv_rope(x, w_qkv, q_out, cos, sin, pairing: int, nh: int, nkv: int, hd: int,
                     tok_pos, tok_seq, seq_slot, table, kc, vc, block_tokens: int,
                     write_cache: bool) -> None:
    """q|k|v product on the tensor cores with rotary and the cache write in its epilogue."""
    _need(x, "x", torch.bfloat16, 2); _need(w_qkv, "w_qkv", torch.bfloat16, 2)
    _need(q_out, "q", torch.bfloat16, 2)
    M, K = x.shape
    if tuple(w_qkv.shape) != ((nh + 2 * nkv) * hd, K) or q_out.shape[0] != M:
        raise KernelError("gemm_tc_qkv_rope: shapes do not fit")
    if cos.shape[1] != hd // 2:
        raise KernelError("gemm_tc_qkv_rope: needs rotary_dim == head_dim")
    _check(lib().cretif_gemm_tc_qkv_rope(
        _p(x), _p(w_qkv), _p(q_out), _rows(q_out, "q"), _p(cos), _p(sin), pairing, nh, nkv, hd,
        _p(tok_pos), _p(tok_seq), _p(seq_slot), _p(table), table.stride(0), _p(kc), _p(vc),
        block_tokens, int(write_cache), M, K, _rows(x, "x"), _rows(w_qkv, "w_qkv"),
        _p(fault_word(x.device)), _stream()), "gemm_tc_qkv_rope")


def set_tc_pair(mode: int) -> int:
    """(For tests that run both.)  The tensor-core product with two CTAs on a tile: -1 where
    the launcher sees fit (the default), 0 never, 1 wherever the kernel takes the product.
    Returns the old setting."""
    return int(lib().cretif_set_tc_pair(int(mode)))


def set_tc_bulk_add(on: bool) -> bool:
    """(For tests that run both.)  Whether the tensor-core product adds into a float32 matrix
    through TMA where it can (the default).  Returns the old setting."""
    return bool(lib().cretif_set_tc_bulk_add(1 if on else 0))


def set_prefill_pairing(mode: int) -> int:
    """(For tests that run all.)  Which prefill attention kernel takes head sizes up to 64
    without a window: -1 as the launcher sees fit (the default), 0 the kernel with two threads
    per row, 1 a thread per row and two query tiles per CTA, 2 a thread per row and one tile
    per CTA whose key steps two groups of warps share.  Returns the old setting."""
    return int(lib().cretif_set_prefill_pairing(int(mode)))


def attn_prefill_supported(hd: int, block_tokens: int) -> bool:
    return block_tokens == 64 and hd % 16 == 0 and 16 <= hd <= 128


def attn_prefill(qkv, out, kc, vc, table, cu_seqlens, seq_start, seq_slot, nh: int, nkv: int,
                 hd: int, scale: float, window: int, block_tokens: int, B: int, max_new: int,
                 fault) -> None:
    """Causal attention of whole prompts; ``qkv`` rows start with the query heads."""
    _need(qkv, "qkv", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(kc, "k cache", torch.bfloat16, 4); _need(vc, "v cache", torch.bfloat16, 4)
    if (tuple(kc.shape[1:]) != (nkv, block_tokens, hd) or not kc.is_contiguous()
            or not vc.is_contiguous()):
        raise KernelError("attn_prefill: cache must be contiguous [blocks, kv_heads, 64, head_dim]")
    _check(lib().cretif_attn_prefill_tc(
        _p(qkv), _rows(qkv, "qkv"), qkv.shape[0], _p(out), _rows(out, "out"), _p(kc), _p(vc),
        ctypes.c_longlong(kc.shape[0]), _p(table), table.stride(0), _p(cu_seqlens), _p(seq_start),
        _p(seq_slot), nh, nkv, hd, ctypes.c_float(scale), window, block_tokens, B, max_new,
        _p(fault), _stream()), "attn_prefill_tc")
