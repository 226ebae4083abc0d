"""The decode-attention entry point for callers that cannot allocate device memory.

Some users of the kernel library run where cudaMalloc is not an option: inside a host
application that owns the device heap, in a real-time loop that must not touch the
allocator, or with all device memory already taken.  For them the library exports
``cretif_attn_decode_noalloc``, whose scratch is a fixed 4 MiB array inside the library
instead of caller-provided buffers.  This test calls it through its exported C symbol, as
such a caller would, twice in a row with different inputs (the second call finds the first
call's leftovers in the shared array), and compares each result with the ordinary entry
point's and with the attention formula in float64.  Further calls use more key ranges with
a sliding window, and a shape that fills the fixed array almost to its end; shapes beyond
the array are refused.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make_case(seed, lens, nh, nkv, hd):
    """Random block cache with a shuffled block table, queries at the last positions."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    rng = np.random.default_rng(seed)
    B = len(lens)
    per = [-(-n // 64) for n in lens]
    n_blocks = sum(per) + 2
    order = rng.permutation(n_blocks)
    table = np.full((B, max(per)), -1, dtype=np.int32)
    o = 0
    for b in range(B):
        table[b, :per[b]] = order[o:o + per[b]]
        o += per[b]
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(DEV)
    return {
        "q": mk(B, nh * hd), "k": mk(n_blocks, nkv, 64, hd), "v": mk(n_blocks, nkv, 64, hd),
        "table": torch.from_numpy(table).to(DEV),
        "pos": torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV),
        "seq": torch.arange(B, dtype=torch.int32, device=DEV),
        "slot": torch.arange(B, dtype=torch.int32, device=DEV),
    }


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _formula(case, lens, nh, nkv, hd, scale, window=0):
    """softmax(q·k·scale)·v in float64 over each sequence's keys, gathered from the blocks."""
    q = case["q"].double().cpu().reshape(len(lens), nh, hd)
    k, v, table = case["k"].double().cpu(), case["v"].double().cpu(), case["table"].cpu()
    out = torch.zeros(len(lens), nh, hd, dtype=torch.float64)
    g = nh // nkv
    for b, n in enumerate(lens):
        blocks = table[b, : -(-n // 64)].long()
        kb = k[blocks].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]      # [nkv, n, hd]
        vb = v[blocks].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]
        lo = max(0, n - window) if window > 0 else 0          # the query sits at n - 1
        for h in range(nh):
            s = (kb[h // g, lo:] @ q[b, h]) * scale
            out[b, h] = torch.softmax(s, dim=0) @ vb[h // g, lo:]
    return out.reshape(len(lens), nh * hd)


def _err(got, want):
    return (got.double().cpu() - want.double().cpu()).abs().max().item() / \
        want.double().abs().max().item()


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from cretif_b200.csrc import ops
    lib = ops.lib()
    fn = lib.cretif_attn_decode_noalloc            # the exported C symbol
    fn.restype = ctypes.c_int
    lib.cretif_attn_decode_noalloc_capacity.restype = ctypes.c_uint
    assert lib.cretif_attn_decode_noalloc_capacity() == 4 << 20
    nh, nkv, hd, splits = 9, 3, 64, 7
    scale = 1.0 / math.sqrt(hd)
    fault = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(case, n_splits, B=None, window=0, heads=(nh, nkv, hd)):
        h, kv, d = heads
        B = case["q"].shape[0] if B is None else B
        out = torch.zeros(case["q"].shape[0], h * d, dtype=torch.bfloat16, device=DEV)
        rc = fn(_ptr(case["q"]), h * d, _ptr(out), h * d, _ptr(case["k"]), _ptr(case["v"]),
                ctypes.c_longlong(case["k"].shape[0]), _ptr(case["table"]),
                case["table"].stride(0), _ptr(case["pos"]), _ptr(case["seq"]), _ptr(case["slot"]),
                h, kv, d, ctypes.c_float(1.0 / math.sqrt(d)), window, 64, B, n_splits,
                _ptr(fault), stream)
        return rc, out

    # two calls in a row, other inputs the second time
    for seed, lens in ((1, [300, 64, 1, 2000]), (2, [77, 1500, 513])):
        case = _make_case(seed, lens, nh, nkv, hd)
        rc, got = call(case, splits)
        assert rc == 0
        want = torch.empty_like(got)
        ops.attn_decode(case["q"], want, case["k"], case["v"], case["table"], case["pos"],
                        case["seq"], case["slot"], nh, nkv, hd, scale, 0, 64, splits, fault)
        torch.cuda.synchronize()
        assert fault.item() == 0
        assert _err(got, want) <= 1e-2            # the tolerance of the other attention tests
        assert _err(got, _formula(case, lens, nh, nkv, hd, scale)) <= 1e-2

    # more ranges than some sequences have blocks, and a window that hides all but 100 keys
    lens = [900, 130, 64, 5]
    case = _make_case(4, lens, nh, nkv, hd)
    rc, got = call(case, 16, window=100)
    torch.cuda.synchronize()
    assert rc == 0 and fault.item() == 0
    assert _err(got, _formula(case, lens, nh, nkv, hd, scale, window=100)) <= 1e-2

    # a shape that takes the fixed array almost to its end: 4,095 of 4,096 counters and
    # 1,031,940 of 1,044,480 floats of partial results
    heads = (3, 3, 16)
    lens = (np.random.default_rng(5).integers(1, 130, size=1365)).tolist()
    case = _make_case(5, lens, *heads)
    rc, got = call(case, 14, heads=heads)
    torch.cuda.synchronize()
    assert rc == 0 and fault.item() == 0
    assert _err(got, _formula(case, lens, *heads, 1.0 / math.sqrt(16))) <= 1e-2
    rc, out = call(case, 15, heads=heads)  # one range more no longer fits
    assert rc == -1 and out.abs().max().item() == 0.0

    # sizes beyond the fixed array are refused, and nothing is launched
    case = _make_case(3, [10, 10], nh, nkv, hd)
    rc, out = call(case, 64, B=2000)       # 2000 * 3 counters > 4096
    assert rc == -1 and out.abs().max().item() == 0.0
    rc, out = call(case, 64, B=1000)       # 1000 * 9 * 64 * 66 floats > 4 MiB
    assert rc == -1 and out.abs().max().item() == 0.0
