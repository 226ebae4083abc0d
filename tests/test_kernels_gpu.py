"""Each kernel alone against a plain float32/float64 torch formula of the same operation,
at sizes other than the engine's (odd widths, head sizes in steps of 16, tails)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from cretif_b200.csrc import ops as _ops
    _ops.lib()
    return _ops


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, rel):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= rel, f"relative error {err:.3e} > {rel:.1e}"


# ------------------------------------------------------------------ matrix products
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 77), (70, 65, 129), (257, 96, 200)])
def test_gemm_simt_f32(ops, M, N, K):
    a, w = rnd(M, K), rnd(N, K, seed=1)
    c = torch.empty(M, N, device=DEV)
    ops.gemm_simt(a, w, c)
    close(c, a.double() @ w.double().T, 2e-6)
    base = rnd(M, N, seed=2)
    c2 = base.clone()
    ops.gemm_simt(a, w, c2, accumulate=True)
    close(c2, base.double() + a.double() @ w.double().T, 2e-6)


@pytest.mark.parametrize("M,N,K", [(2, 33, 40), (65, 70, 136)])
def test_gemm_simt_bf16(ops, M, N, K):
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    want = a.double() @ w.double().T
    c32 = torch.empty(M, N, device=DEV)
    ops.gemm_simt(a, w, c32)
    close(c32, want, 1e-5)
    c16 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm_simt(a, w, c16)
    close(c16, want, 5e-3)


@pytest.mark.parametrize("M,N,K", [(1, 16, 32), (1, 1000, 576), (3, 50, 40), (8, 333, 1544),
                                   (9, 96, 104), (17, 64, 72), (33, 200, 256), (64, 129, 520)])
def test_gemm_skinny(ops, M, N, K):
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    want = x.double() @ w.double().T
    assert ops.gemv_supported(x, w, torch.empty(M, N, device=DEV))
    c = torch.empty(M, N, device=DEV)
    ops.gemv_bf16(x, w, c)
    close(c, want, 1e-5)
    base = rnd(M, N, seed=3)
    c2 = base.clone()
    ops.gemv_bf16(x, w, c2, accumulate=True)
    close(c2, base.double() + want, 1e-5)
    cb = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemv_bf16(x, w, cb)
    close(cb, want, 5e-3)


def test_gemm_skinny_strided_rows(ops):
    """Rows of x may be a slice of a wider buffer (its row stride a multiple of 8)."""
    buf = rnd(5, 256, dtype=torch.bfloat16)
    x = buf[:, 64:64 + 72]
    w = rnd(40, 72, dtype=torch.bfloat16, seed=1)
    c = torch.empty(5, 40, device=DEV)
    ops.gemv_bf16(x, w, c)
    close(c, x.double() @ w.double().T, 1e-5)


def test_gemm_skinny_refuses_unaligned(ops):
    x, w = rnd(2, 20, dtype=torch.bfloat16), rnd(8, 20, dtype=torch.bfloat16)
    assert not ops.gemv_supported(x, w, torch.empty(2, 8, device=DEV))
    with pytest.raises(ops.KernelError):
        ops.gemv_bf16(x, w, torch.empty(2, 8, device=DEV))


@pytest.fixture(params=[4, 8], ids=["4-epilogue-warps", "8-epilogue-warps"])
def tc_epilogue(request, ops):
    """The tensor-core product drains an accumulator with four warps (a thread per row) or
    with eight (two threads per row, half of the columns each); a launch chooses by its size.
    Tests of that kernel run both ways."""
    old = ops.set_tc_epilogue_warps(request.param)
    yield request.param
    ops.set_tc_epilogue_warps(old)


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 64, 128), (128, 64, 128, 64), (256, 256, 256, 256),
                                      (2048, 960, 576, 0), (300, 200, 72, 0), (129, 65, 136, 64),
                                      (70, 1000, 1544, 128), (1000, 3072, 576, 256),
                                      (513, 576, 1536, 0), (300, 576, 72, 192),
                                      (1000, 960, 576, 192), (130, 200, 136, 192),
                                      # enough rows that a width of 3 x 192 picks 192 itself
                                      (19000, 576, 136, 0)])
def test_gemm_tc(ops, tc_epilogue, M, N, K, bn):
    """The tcgen05 kernel against float64, tails in every dimension."""
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    want = x.double() @ w.double().T
    ldc = -(-N // 8) * 8
    fault = ops.fault_word(DEV)
    fault.zero_()
    c = torch.full((M, ldc), 7.0, device=DEV)[:, :N]
    assert ops.gemm_tc_supported(x, w, c)
    ops.gemm_tc(x, w, c, bn=bn)
    torch.cuda.synchronize()
    assert fault.item() == 0
    close(c, want, 1e-5)
    # added into a float32 matrix: by the epilogue's threads, and (a row pitch of whole 16
    # bytes) through TMA, which clips the tile at both edges; what lies beside the matrix in
    # its rows' padding stays as it is
    base = rnd(M, ldc, seed=3)
    for bulk in (False, True):
        old = ops.set_tc_bulk_add(bulk)
        before = ops.variant_counts()["tc_bulk_add"]
        full = base.clone()
        c2 = full[:, :N]
        ops.gemm_tc(x, w, c2, accumulate=True, bn=bn)
        ops.set_tc_bulk_add(old)
        close(c2, base[:, :N].double() + want, 1e-5)
        assert torch.equal(full[:, N:], base[:, N:])
        took = ops.variant_counts()["tc_bulk_add"] > before
        assert took == (bulk and ldc % 4 == 0)
    cb = torch.empty((M, ldc), device=DEV, dtype=torch.bfloat16)[:, :N]
    ops.gemm_tc(x, w, cb, bn=bn)
    close(cb, want, 5e-3)
    assert fault.item() == 0


@pytest.mark.parametrize("M,N,K,bn", [(256, 256, 64, 256), (1000, 512, 136, 256), (300, 576, 72, 192),
                                      (130, 960, 200, 192), (2100, 2048, 264, 256)])
def test_gemm_tc_with_two_ctas_on_a_tile(ops, M, N, K, bn):
    """The float32 add with a cluster of two CTAs on each tile of 256 rows (cta_group::2)
    against float64, tails in M and K, and the same numbers as the single-CTA kernel."""
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1)
    base = rnd(M, N, seed=3)
    want = base.double() + x.double() @ w.double().T
    fault = ops.fault_word(DEV)
    fault.zero_()
    got = {}
    for mode in (0, 1):
        old = ops.set_tc_pair(mode)
        before = ops.variant_counts()["tc_pair"]
        c = base.clone()
        ops.gemm_tc(x, w, c, accumulate=True, bn=bn)
        ops.set_tc_pair(old)
        torch.cuda.synchronize()
        assert (ops.variant_counts()["tc_pair"] > before) == (mode == 1)
        close(c, want, 1e-5)
        got[mode] = c
    assert fault.item() == 0
    assert torch.equal(got[0], got[1])


@pytest.mark.parametrize("M,I,K", [(256, 128, 64), (2200, 4224, 72), (300, 1536, 576)])
def test_gemm_tc_silu_with_two_ctas_on_a_tile(ops, M, I, K):
    x = rnd(M, K, dtype=torch.bfloat16)
    gate = rnd(I, K, dtype=torch.bfloat16, seed=1, scale=0.3)
    up = rnd(I, K, dtype=torch.bfloat16, seed=2, scale=0.3)
    w = _interleave(gate, up)
    g = (x.double() @ gate.double().T).to(torch.bfloat16).double()
    u = (x.double() @ up.double().T).to(torch.bfloat16).double()
    fault = ops.fault_word(DEV)
    fault.zero_()
    old = ops.set_tc_pair(1)
    before = ops.variant_counts()["tc_pair"]
    act = torch.zeros(M, I, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc_silu(x, w, act)
    ops.set_tc_pair(old)
    torch.cuda.synchronize()
    assert ops.variant_counts()["tc_pair"] > before and fault.item() == 0
    close(act, g / (1 + torch.exp(-g)) * u, 1e-2)


# ------------------------------------------------------------------ fused decode projections
@pytest.fixture(params=[(1 << 20, 1 << 40, 4), (1 << 20, 1 << 40, 1), (64, 0, 4)],
                ids=["registers", "registers-no-cluster", "streamed"])
def fused_variant(request, ops):
    """The fused product has two bodies: weights through registers (narrow, small matrices)
    and through a shared-memory ring (wide or large ones).  Every fused test runs with
    thresholds that keep the test matrices in registers, and with ones that send them
    through the ring; the register body with more than eight rows runs with its norm
    prologue shared by a thread-block cluster, and with every CTA on its own."""
    old_bytes = ops.stream_min_bytes()
    old_k = ops.set_stream_min_k(*request.param[:2])
    old_cluster = ops.set_fused_cluster(request.param[2])
    yield request.param[0]
    ops.set_stream_min_k(old_k, old_bytes)
    ops.set_fused_cluster(old_cluster)


def _norm_bf16(h, w, eps, rows=None):
    """bf16(rmsnorm(h[rows])) as the fused prologue stores it, in float64."""
    x = h.double().cpu()
    if rows is not None:
        x = x[rows]
    n = x * w.double().cpu() / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return n.to(torch.bfloat16).double()


@pytest.mark.parametrize("M,N,K", [(1, 48, 64), (8, 1000, 576), (5, 50, 104), (16, 333, 200),
                                   (17, 96, 72), (32, 130, 576), (8, 200, 2048), (3, 64, 1544),
                                   (16, 48, 8192), (13, 77, 3000),
                                   # more than 32 rows: groups of rows in one launch
                                   (33, 130, 576), (40, 130, 576), (57, 100, 960), (64, 96, 104),
                                   (100, 50, 200), (128, 96, 136)])
def test_fused_norm_linear_and_add(ops, fused_variant, M, N, K):
    eps = 1e-5
    h, nw = rnd(M + 3, K), rnd(K, seed=1) * 0.1 + 1
    w = rnd(N, K, dtype=torch.bfloat16, seed=2)
    out = torch.empty(M, N, device=DEV)
    if ops.fused_supported(M, K, w):          # the normed rows must fit in shared memory
        ops.fused_norm_linear(h[:M].contiguous(), nw, eps, w, out)
        close(out, _norm_bf16(h[:M], nw, eps) @ w.double().cpu().T, 3e-3)
        rows = torch.tensor([(3 * i + 2) % (M + 3) for i in range(M)], dtype=torch.int32,
                            device=DEV)
        ops.fused_norm_linear(h, nw, eps, w, out, rows=rows)
        close(out, _norm_bf16(h, nw, eps, rows.cpu().long()) @ w.double().cpu().T, 3e-3)
    else:
        assert (M, K) == (16, 8192)
    assert ops.fused_supported(M, K, w, norm=False)
    x = rnd(M, K, dtype=torch.bfloat16, seed=4)
    base = rnd(M, N, seed=5)
    acc = base.clone()
    ops.fused_linear_add(x, w, acc)
    close(acc, base.double().cpu() + x.double().cpu() @ w.double().cpu().T, 1e-5)


@pytest.mark.parametrize("M,I,K", [(1, 8, 64), (8, 1536, 576), (7, 173, 104), (20, 256, 96),
                                   (8, 512, 2048), (12, 72, 1032), (50, 256, 96),
                                   (64, 1536, 576), (33, 1536, 576), (90, 200, 104)])
def test_fused_gate_up_silu_equals_the_separate_kernels(ops, fused_variant, M, I, K):
    eps = 1e-6
    h, nw = rnd(M, K), rnd(K, seed=1) * 0.1 + 1
    w = rnd(2 * I, K, dtype=torch.bfloat16, seed=2, scale=0.3)
    act = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    ops.fused_gate_up_silu(h, nw, eps, w, act)
    n = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
    ops.add_rmsnorm(h.clone(), None, nw, n, eps)
    gu = torch.empty(M, 2 * I, device=DEV, dtype=torch.bfloat16)
    ops.gemm_simt(n, w, gu)
    want = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    ops.silu_mul(gu, want)
    close(act, want, 1e-2)                     # the same roundings; sums in another order
    x = _norm_bf16(h, nw, eps)
    g = (x @ w[:I].double().cpu().T).to(torch.bfloat16).double()
    u = (x @ w[I:].double().cpu().T).to(torch.bfloat16).double()
    close(act, g / (1 + torch.exp(-g)) * u, 1e-2)


@pytest.mark.parametrize("pairing", [0, 1])
@pytest.mark.parametrize("many", [0, 45, 110], ids=["6tokens", "45tokens", "110tokens"])
@pytest.mark.parametrize("nh,nkv,hd,K", [(4, 2, 16, 64), (9, 3, 64, 576), (3, 1, 32, 96),
                                         (5, 5, 48, 104), (4, 4, 64, 2048)])
def test_fused_qkv_rope_equals_the_separate_kernels(ops, fused_variant, pairing, many, nh, nkv,
                                                    hd, K):
    eps, theta, P = 1e-5, 10000.0, 256
    lens = [25, 70, 130]
    j = torch.arange(hd // 2, dtype=torch.float64)
    ang = torch.arange(P, dtype=torch.float64)[:, None] / theta ** (2 * j / hd)[None, :]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    if many == 45:    # 33 to 64 tokens: two groups of rows in one launch
        qpos = list(range(10, 25)) + list(range(50, 65)) + list(range(115, 130))
        qseq = [0] * 15 + [1] * 15 + [2] * 15
    elif many:        # more than 64 tokens: four groups
        qpos = list(range(5, 25)) + list(range(30, 70)) + list(range(80, 130))
        qseq = [0] * 20 + [1] * 40 + [2] * 50
    else:
        qpos = [4, 3, 64, 69, 129, 0]
        qseq = [0, 0, 1, 1, 2, 2]
    T = len(qpos)
    pos_t = torch.tensor(qpos, dtype=torch.int32, device=DEV)
    seq_t = torch.tensor(qseq, dtype=torch.int32, device=DEV)
    h, nw = rnd(T, K), rnd(K, seed=1) * 0.1 + 1
    w = rnd((nh + 2 * nkv) * hd, K, dtype=torch.bfloat16, seed=2, scale=0.3)
    fault = torch.zeros(1, dtype=torch.int32, device=DEV)
    # separate kernels
    ca = ToyCache(lens, nkv, hd, torch.bfloat16, seed=3)
    n = torch.empty(T, K, device=DEV, dtype=torch.bfloat16)
    ops.add_rmsnorm(h.clone(), None, nw, n, eps)
    qkv = torch.empty(T, (nh + 2 * nkv) * hd, device=DEV, dtype=torch.bfloat16)
    ops.gemm_simt(n, w, qkv)
    ops.rope_kv_append(qkv, cos, sin, pairing, hd, nh, nkv, hd, pos_t, seq_t, ca.seq_slot,
                       ca.table, ca.k, ca.v, 64, True, fault)
    # fused
    cb = ToyCache(lens, nkv, hd, torch.bfloat16, seed=3)
    q = torch.zeros(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    ops.fused_qkv_rope(h, nw, eps, w, q, cos, sin, pairing, nh, nkv, hd, pos_t, seq_t,
                       cb.seq_slot, cb.table, cb.k, cb.v, 64, True, fault)
    assert fault.item() == 0
    close(q, qkv[:, :nh * hd], 1e-2)
    close(cb.k, ca.k, 1e-2)
    close(cb.v, ca.v, 1e-2)
    # and writing can be switched off (a visit that borrows another visit's cache)
    cc = ToyCache(lens, nkv, hd, torch.bfloat16, seed=3)
    before = cc.k.clone()
    ops.fused_qkv_rope(h, nw, eps, w, q, cos, sin, pairing, nh, nkv, hd, pos_t, seq_t,
                       cc.seq_slot, cc.table, cc.k, cc.v, 64, False, fault)
    assert torch.equal(cc.k, before)


# ------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("T,H", [(1, 10), (5, 100), (3, 576), (2, 3000), (4, 6), (2, 8200)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(ops, T, H, out_dtype):
    eps = 3e-6
    h, d, w = rnd(T, H), rnd(T, H, seed=1), rnd(H, seed=2) + 1
    want_h = h.double() + d.double()
    want_n = want_h * w.double() / torch.sqrt((want_h ** 2).mean(-1, keepdim=True) + eps)
    out = torch.empty(T, H, device=DEV, dtype=out_dtype)
    h2 = h.clone()
    ops.add_rmsnorm(h2, d, w, out, eps)
    close(h2, want_h, 1e-7)
    close(out, want_n, 1e-5 if out_dtype == torch.float32 else 5e-3)
    # no delta: h untouched
    h3 = h.clone()
    ops.add_rmsnorm(h3, None, w, out, eps)
    assert torch.equal(h3, h)
    want0 = h.double() * w.double() / torch.sqrt((h.double() ** 2).mean(-1, keepdim=True) + eps)
    close(out, want0, 1e-5 if out_dtype == torch.float32 else 5e-3)
    # gathered rows with a bfloat16 delta: the stream is not written
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    db = d.to(torch.bfloat16)
    out2 = torch.empty(2, H, device=DEV, dtype=out_dtype)
    h4 = h.clone()
    ops.add_rmsnorm(h4, db, w, out2, eps, rows=rows)
    assert torch.equal(h4, h)
    wh = h.double() + db.double()
    wn = (wh * w.double() / torch.sqrt((wh ** 2).mean(-1, keepdim=True) + eps))[[T - 1, 0]]
    close(out2, wn, 1e-5 if out_dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(ops, dtype):
    T, I = 5, 173
    gu = rnd(T, 2 * I, dtype=dtype, scale=3.0)
    act = torch.empty(T, I, device=DEV, dtype=dtype)
    ops.silu_mul(gu, act)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    close(act, g / (1 + torch.exp(-g)) * u, 1e-6 if dtype == torch.float32 else 5e-3)
    # gate and up columns alternating in groups of 16
    I, b = 96, 16
    gu = rnd(T, 2 * I, dtype=dtype, scale=3.0)
    act = torch.empty(T, I, device=DEV, dtype=dtype)
    ops.silu_mul(gu, act, b)
    blocks = gu.double().reshape(T, I // b, 2, b)
    g, u = blocks[:, :, 0, :].reshape(T, I), blocks[:, :, 1, :].reshape(T, I)
    close(act, g / (1 + torch.exp(-g)) * u, 1e-6 if dtype == torch.float32 else 5e-3)


def _interleave(gate, up, b=64):
    I = gate.shape[0]
    return torch.stack([gate.reshape(I // b, b, -1), up.reshape(I // b, b, -1)], dim=1).reshape(
        2 * I, -1).contiguous()


@pytest.mark.parametrize("M,I,K", [(128, 64, 64), (300, 1536, 576), (70, 192, 104), (2048, 256, 96),
                                   (2200, 4288, 72)])     # wide tiles of two gate|up pairs
def test_gemm_tc_silu(ops, tc_epilogue, M, I, K):
    x = rnd(M, K, dtype=torch.bfloat16)
    gate = rnd(I, K, dtype=torch.bfloat16, seed=1, scale=0.3)
    up = rnd(I, K, dtype=torch.bfloat16, seed=2, scale=0.3)
    w = _interleave(gate, up)
    fault = ops.fault_word(DEV)
    fault.zero_()
    g = (x.double() @ gate.double().T).to(torch.bfloat16).double()
    u = (x.double() @ up.double().T).to(torch.bfloat16).double()
    for bulk in (False, True):       # stored by the epilogue's threads, and through TMA
        old = ops.set_tc_bulk_add(bulk)
        act = torch.zeros(M, I, device=DEV, dtype=torch.bfloat16)
        ops.gemm_tc_silu(x, w, act)
        ops.set_tc_bulk_add(old)
        torch.cuda.synchronize()
        assert fault.item() == 0
        close(act, g / (1 + torch.exp(-g)) * u, 1e-2)
    # the few-token kernel reads the same interleaved matrix
    h, nw = rnd(8, K), rnd(K, seed=3) * 0.1 + 1
    a2 = torch.empty(8, I, device=DEV, dtype=torch.bfloat16)
    ops.fused_gate_up_silu(h, nw, 1e-5, w, a2, 64)
    a3 = torch.empty(8, I, device=DEV, dtype=torch.bfloat16)
    ops.fused_gate_up_silu(h, nw, 1e-5, torch.cat([gate, up]).contiguous(), a3, 0)
    close(a2, a3, 1e-2)


@pytest.mark.parametrize("pairing", [0, 1])
@pytest.mark.parametrize("nh,nkv,hd,K,long", [
    (9, 3, 64, 576, False), (2, 1, 128, 96, False), (3, 3, 64, 72, False),
    # so many heads that a tile takes two of them (and the last tile only one)
    (101, 25, 64, 72, False),
    # so many tokens that a tile takes three heads (15 heads = 5 tiles of 192 columns)
    (9, 3, 64, 72, True)])
def test_gemm_tc_qkv_rope_equals_the_separate_kernels(ops, tc_epilogue, pairing, nh, nkv, hd, K,
                                                      long):
    theta, P = 10000.0, 4096 if long else 512
    lens = [200, 70, 333]
    news = [200, 70, 150]                     # the third sequence continues at 183
    if long:
        lens, news = [4000, 70, 3900], [4000, 70, 3800]
    before_192 = ops.variant_counts()["tc192"]
    j = torch.arange(hd // 2, dtype=torch.float64)
    ang = torch.arange(P, dtype=torch.float64)[:, None] / theta ** (2 * j / hd)[None, :]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    qpos, qseq = [], []
    for b, (n, m) in enumerate(zip(lens, news)):
        qpos += list(range(n - m, n)); qseq += [b] * m
    T = len(qpos)
    pos_t = torch.tensor(qpos, dtype=torch.int32, device=DEV)
    seq_t = torch.tensor(qseq, dtype=torch.int32, device=DEV)
    x = rnd(T, K, dtype=torch.bfloat16)
    w = rnd((nh + 2 * nkv) * hd, K, dtype=torch.bfloat16, seed=2, scale=0.3)
    fault = ops.fault_word(DEV)
    fault.zero_()
    ca = ToyCache(lens, nkv, hd, torch.bfloat16, seed=3)
    qkv = torch.empty(T, (nh + 2 * nkv) * hd, device=DEV, dtype=torch.bfloat16)
    ops.gemm_simt(x, w, qkv)
    ops.rope_kv_append(qkv, cos, sin, pairing, hd, nh, nkv, hd, pos_t, seq_t, ca.seq_slot,
                       ca.table, ca.k, ca.v, 64, True, fault)
    cb = ToyCache(lens, nkv, hd, torch.bfloat16, seed=3)
    q = torch.zeros(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc_qkv_rope(x, w, q, cos, sin, pairing, nh, nkv, hd, pos_t, seq_t, cb.seq_slot,
                         cb.table, cb.k, cb.v, 64, True)
    torch.cuda.synchronize()
    assert fault.item() == 0
    assert (ops.variant_counts()["tc192"] > before_192) == long
    close(q, qkv[:, :nh * hd], 1e-2)
    close(cb.k, ca.k, 1e-2)
    close(cb.v, ca.v, 1e-2)
    cc = ToyCache(lens, nkv, hd, torch.bfloat16, seed=3)
    before = cc.k.clone()
    ops.gemm_tc_qkv_rope(x, w, q, cos, sin, pairing, nh, nkv, hd, pos_t, seq_t, cc.seq_slot,
                         cc.table, cc.k, cc.v, 64, False)
    assert torch.equal(cc.k, before)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(ops, dtype):
    table = rnd(50, 37, dtype=dtype)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 37, device=DEV)
    fault = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed_rows(table, ids, out, fault)
    assert torch.equal(out, table[ids.long()].float())
    assert fault.item() == 0
    bad = torch.tensor([3, 50], dtype=torch.int32, device=DEV)
    out2 = torch.ones(2, 37, device=DEV)
    ops.embed_rows(table, bad, out2, fault)
    assert fault.item() & 1 and out2[1].abs().max().item() == 0.0


# ------------------------------------------------------------------ cache helpers
class ToyCache:
    """A block cache with a shuffled block table, as the kernels see it."""

    def __init__(self, lens, nkv, hd, dtype, bt=64, seed=0, spare=3):
        self.lens, self.nkv, self.hd, self.bt = lens, nkv, hd, bt
        B = len(lens)
        per = [-(-n // bt) for n in lens]
        n_blocks = sum(per) + spare
        rng = np.random.default_rng(seed)
        order = rng.permutation(n_blocks)
        self.slots = rng.permutation(B + 2)[:B]              # slots are not 0..B-1
        table = np.full((B + 2, max(per) + 1), -1, dtype=np.int32)
        o = 0
        for b in range(B):
            table[self.slots[b], :per[b]] = order[o:o + per[b]]
            o += per[b]
        self.table_host = table
        self.table = torch.from_numpy(table).to(DEV)
        self.k = rnd(n_blocks, nkv, bt, hd, dtype=dtype, seed=seed + 1)
        self.v = rnd(n_blocks, nkv, bt, hd, dtype=dtype, seed=seed + 2)
        self.seq_slot = torch.from_numpy(self.slots.astype(np.int32)).to(DEV)

    def keys(self, b, n):
        """K and V of sequence b, positions 0..n-1: [n, nkv, hd] float64."""
        ks, vs = [], []
        for p in range(n):
            blk = self.table_host[self.slots[b], p // self.bt]
            ks.append(self.k[blk, :, p % self.bt, :])
            vs.append(self.v[blk, :, p % self.bt, :])
        return torch.stack(ks).double().cpu(), torch.stack(vs).double().cpu()


def plain_attention(q, k, v, scale, qpos, window=0):
    """q [nq, nh, hd] at positions qpos, k/v [n, nkv, hd] → [nq, nh, hd] (float64)."""
    nq, nh, hd = q.shape
    g = nh // k.shape[1]
    out = torch.zeros(nq, nh, hd, dtype=torch.float64)
    for i in range(nq):
        p = qpos[i]
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(nh):
            s = (k[lo:p + 1, h // g, :] @ q[i, h]) * scale
            w = torch.softmax(s, dim=0)
            out[i, h] = w @ v[lo:p + 1, h // g, :]
    return out


ATTN_CASES = [  # nh, nkv, hd, lens
    (4, 2, 16, [1, 64, 65, 200]),
    (3, 1, 32, [17, 129]),
    (5, 5, 48, [70, 3]),
    (8, 1, 64, [300]),
    (6, 2, 128, [130, 64]),
    (2, 2, 256, [90]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,lens", ATTN_CASES)
@pytest.mark.parametrize("window", [0, 40])
def test_attn_simt_decode_and_prefill(ops, dtype, nh, nkv, hd, lens, window):
    scale = 0.37 / math.sqrt(hd)
    cache = ToyCache(lens, nkv, hd, dtype)
    B = len(lens)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    # decode shape: one query per sequence at its last position
    q = rnd(B, nh * hd, dtype=dtype, seed=5)
    out = torch.empty(B, nh * hd, device=DEV, dtype=dtype)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    ops.attn_simt(q, out, cache.k, cache.v, cache.table, pos, seq, cache.seq_slot, nh, nkv, hd,
                  scale, window, 64)
    for b, n in enumerate(lens):
        k, v = cache.keys(b, n)
        want = plain_attention(q[b].double().cpu().reshape(1, nh, hd), k, v, scale, [n - 1], window)
        close(out[b].reshape(1, nh, hd), want, tol)
    # prefill shape: the last min(n, 20) positions of every sequence as queries
    qpos, qseq = [], []
    for b, n in enumerate(lens):
        for p in range(max(0, n - 20), n):
            qpos.append(p); qseq.append(b)
    T = len(qpos)
    q = rnd(T, nh * hd + 16, dtype=dtype, seed=6)[:, :nh * hd]        # strided rows
    out = torch.empty(T, nh * hd, device=DEV, dtype=dtype)
    ops.attn_simt(q, out, cache.k, cache.v, cache.table,
                  torch.tensor(qpos, dtype=torch.int32, device=DEV),
                  torch.tensor(qseq, dtype=torch.int32, device=DEV), cache.seq_slot, nh, nkv, hd,
                  scale, window, 64)
    for b, n in enumerate(lens):
        k, v = cache.keys(b, n)
        idx = [i for i in range(T) if qseq[i] == b]
        want = plain_attention(q[idx].double().cpu().reshape(len(idx), nh, hd), k, v, scale,
                               [qpos[i] for i in idx], window)
        close(out[idx].reshape(len(idx), nh, hd), want, tol)


@pytest.mark.parametrize("nh,nkv,hd,lens", ATTN_CASES + [(9, 3, 64, [2048, 700, 1, 4096])])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("simt", [False, True])
def test_attn_decode_split(ops, nh, nkv, hd, lens, window, splits, simt):
    """Both decode kernels (tensor-core for head sizes up to 128, CUDA-core for all)."""
    ops.decode_attention_simt_only(simt)
    try:
        _attn_decode_split(ops, nh, nkv, hd, lens, window, splits)
    finally:
        ops.decode_attention_simt_only(False)


@pytest.mark.parametrize("nh,nkv,hd,lens", [c for c in ATTN_CASES if c[2] <= 128]
                         + [(9, 3, 64, [2048, 700, 1, 4096]), (16, 2, 128, [1000, 3])])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_attn_decode_cluster(ops, nh, nkv, hd, lens, window, splits):
    """The ranges of a sequence as one thread-block cluster, merged through distributed
    shared memory (ranges beyond a short sequence's blocks are empty CTAs of the cluster)."""
    _attn_decode_split(ops, nh, nkv, hd, lens, window, splits, cluster=True)


def test_decode_plan(ops):
    # many sequences or a short context: few ranges, merged inside a cluster
    n, cluster = ops.decode_plan(8, 3, 2100, DEV)
    assert cluster and 1 <= n <= ops.CLUSTER_MAX_RANGES
    n, cluster = ops.decode_plan(64, 3, 2100, DEV)
    assert cluster and n <= 2
    for batch in (1, 5, 8, 12, 16, 24, 32, 48):        # cluster sizes are powers of two
        n, cluster = ops.decode_plan(batch, 3, 2100, DEV)
        assert cluster and n & (n - 1) == 0
    # one long sequence: more ranges than a cluster holds
    n, cluster = ops.decode_plan(1, 1, 64 * 1024, DEV)
    assert not cluster and n > ops.CLUSTER_MAX_RANGES
    # head sizes the tensor-core kernel does not take never get a cluster
    assert ops.decode_plan(8, 3, 2100, DEV, hd=256)[1] is False


def _attn_decode_split(ops, nh, nkv, hd, lens, window, splits, cluster=False):
    scale = 1.0 / math.sqrt(hd)
    cache = ToyCache(lens, nkv, hd, torch.bfloat16, seed=4)
    B = len(lens)
    assert ops.attn_decode_supported(hd, 64, nh // nkv)
    q = rnd(B, nh * hd, dtype=torch.bfloat16, seed=5)
    out = torch.empty(B, nh * hd, device=DEV, dtype=torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    fault = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.attn_decode(q, out, cache.k, cache.v, cache.table, pos, seq, cache.seq_slot, nh, nkv, hd,
                    scale, window, 64, splits, fault, cluster)
    assert fault.item() == 0
    for b, n in enumerate(lens):
        k, v = cache.keys(b, n)
        want = plain_attention(q[b].double().cpu().reshape(1, nh, hd), k, v, scale, [n - 1], window)
        close(out[b].reshape(1, nh, hd), want, 1e-2)


PREFILL_CASES = [  # nh, nkv, hd, lens (cached + new), new tokens per sequence
    (4, 2, 64, [200], [200]),
    (9, 3, 64, [300, 64, 129, 1], [300, 64, 129, 1]),
    (3, 1, 32, [130, 500], [130, 250]),          # the second sequence continues at 250
    (4, 2, 16, [65, 128], [65, 100]),
    (5, 5, 48, [70, 3, 257], [70, 3, 257]),
    (2, 1, 128, [260, 90], [260, 90]),
    (2, 2, 96, [150], [150]),
]


@pytest.fixture(params=[0, 1, 2], ids=["two-threads-per-row", "thread-per-row-two-tiles",
                                       "thread-per-row-split-keys"])
def prefill_pairing(request, ops):
    """The tensor-core prefill attention has a kernel with two threads per row of a tile of 128
    queries (every head size, windows), and one with a thread per row that keeps P and O in
    tensor memory (head sizes up to 64, no window); that one gives a CTA two tiles that share
    a key/value head, or one tile whose key steps its two groups of warps take in turns and
    merge at the end.  A launch chooses by its shape; tests run all three."""
    old = ops.set_prefill_pairing(request.param)
    yield request.param
    ops.set_prefill_pairing(old)


@pytest.mark.parametrize("nh,nkv,hd,lens,news", PREFILL_CASES + [
    # several query tiles and heads per group, so that pairs hold two heads of one tile, two
    # tiles of one head, and a last pair of one item; the second sequence continues at 100
    (9, 3, 64, [700, 500, 129], [700, 400, 129]),
    (4, 1, 48, [390], [390]),
    (2, 2, 16, [1000, 64], [1000, 64])])
@pytest.mark.parametrize("window", [0, 100])
def test_attn_prefill_tc(ops, prefill_pairing, nh, nkv, hd, lens, news, window):
    scale = 1.0 / math.sqrt(hd)
    before = ops.variant_counts()
    cache = ToyCache(lens, nkv, hd, torch.bfloat16, seed=6)
    B = len(lens)
    assert ops.attn_prefill_supported(hd, 64)
    T = sum(news)
    width = (nh + 2 * nkv) * hd
    qkv = rnd(T, width, dtype=torch.bfloat16, seed=7)
    out = torch.zeros(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    cu = np.concatenate([[0], np.cumsum(news)]).astype(np.int32)
    starts = np.array([n - m for n, m in zip(lens, news)], dtype=np.int32)
    fault = ops.fault_word(DEV)
    fault.zero_()
    ops.attn_prefill(qkv, out, cache.k, cache.v, cache.table, torch.from_numpy(cu).to(DEV),
                     torch.from_numpy(starts).to(DEV), cache.seq_slot, nh, nkv, hd, scale, window,
                     64, B, max(news), fault)
    torch.cuda.synchronize()
    assert fault.item() == 0
    now = ops.variant_counts()
    names = ("prefill_attn", "prefill_attn_pair", "prefill_attn_split")
    took = [k for k in names if now[k] > before[k]]
    rows = window == 0 and hd <= 64
    assert took == [names[prefill_pairing if rows else 0]]
    for b, n in enumerate(lens):
        k, v = cache.keys(b, n)
        q = qkv[cu[b]:cu[b + 1], :nh * hd].double().cpu().reshape(news[b], nh, hd)
        want = plain_attention(q, k, v, scale, list(range(starts[b], n)), window)
        close(out[cu[b]:cu[b + 1]].reshape(news[b], nh, hd), want, 1e-2)


def test_attn_prefill_rows_whose_reference_jumps(ops, prefill_pairing):
    """Late in a long prompt a key appears that dominates everything the later queries have
    seen so far (its score exceeds their running reference by far more than 2^8): the kernel
    that keeps its output in tensor memory has to rescale it there, in the middle of the
    sequence.  Queries before that key must not see it.  Against float64."""
    nh, nkv, hd, n = 4, 2, 64, 1000
    late = 700
    cache = ToyCache([n], nkv, hd, torch.bfloat16, seed=31)
    qkv = rnd(n, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=32)
    # queries 800..999 of head 0 and 2 all look like one vector; the key at `late` is 30 x it
    probe = rnd(1, hd, dtype=torch.bfloat16, seed=33)[0]
    for h in (0, 2):
        qkv[800:, h * hd:(h + 1) * hd] = probe
    blk = cache.table_host[cache.slots[0], late // 64]
    for kvh in range(nkv):
        cache.k[blk, kvh, late % 64, :] = (probe.float() * 30).to(torch.bfloat16)
    out = torch.zeros(n, nh * hd, device=DEV, dtype=torch.bfloat16)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    start = torch.zeros(1, dtype=torch.int32, device=DEV)
    fault = ops.fault_word(DEV)
    fault.zero_()
    ops.attn_prefill(qkv, out, cache.k, cache.v, cache.table, cu, start, cache.seq_slot, nh, nkv,
                     hd, 1.0, 0, 64, 1, n, fault)
    torch.cuda.synchronize()
    assert fault.item() == 0
    k, v = cache.keys(0, n)
    q = qkv[:, :nh * hd].double().cpu().reshape(n, nh, hd)
    want = plain_attention(q, k, v, 1.0, list(range(n)))
    close(out.reshape(n, nh, hd), want, 1e-2)
    # the late queries of head 0 return that key's value, the early ones do not
    close(out[900, :hd], cache.v[blk, 0, late % 64, :], 2e-2)
    assert (out[600, :hd].float() - cache.v[blk, 0, late % 64, :].float()).abs().max() > 0.5


@pytest.mark.parametrize("cluster", [False, True])
def test_attn_decode_finds_a_far_key(ops, cluster):
    """One key among thousands is made to dominate; the output must be its value."""
    nh, nkv, hd, n = 4, 2, 64, 3000
    cache = ToyCache([n], nkv, hd, torch.bfloat16, seed=9)
    target = 1234
    blk = cache.table_host[cache.slots[0], target // 64]
    q = rnd(1, nh * hd, dtype=torch.bfloat16, seed=5)
    for kvh in range(nkv):
        cache.k[blk, kvh, target % 64, :] = (q[0, kvh * 2 * hd:kvh * 2 * hd + hd].float() * 40
                                             ).to(torch.bfloat16)
    out = torch.empty(1, nh * hd, device=DEV, dtype=torch.bfloat16)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    fault = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.attn_decode(q, out, cache.k, cache.v, cache.table, pos, seq, cache.seq_slot, nh, nkv, hd,
                    1.0, 0, 64, 7, fault, cluster)
    for h in (0, 2):       # the heads whose own query was copied into the key
        close(out[0, h * hd:(h + 1) * hd], cache.v[blk, h // 2, target % 64, :], 2e-2)


@pytest.mark.parametrize("kernel,splits", [("simt", 1), ("prefill", 1)] + [
    (k, n) for k in ("decode_split", "decode_cluster", "decode_cuda_cores") for n in (1, 3, 16)])
@pytest.mark.parametrize("first_key", [128, 191])       # a block's first and last position
def test_the_edge_of_a_window_with_dominant_keys(ops, kernel, first_key, splits):
    """A query at position 299 with a window that begins at ``first_key``.  The key just
    before the window is made to dominate everything (it must not be seen), the window's
    first key to dominate the rest (it must be): the output is that key's value, and one key
    too many or too few changes it completely.  Random keys alone give diffuse weights under
    which one key at the edge hides inside the tolerance.  With 16 ranges most of them are
    empty, and the leading cache blocks lie wholly outside the window."""
    nh, nkv, hd, n = 4, 2, 64, 300
    pos = n - 1
    window = pos - first_key + 1
    cache = ToyCache([n], nkv, hd, torch.bfloat16, seed=21)
    fault = torch.zeros(1, dtype=torch.int32, device=DEV)
    seq_slot = cache.seq_slot
    if kernel == "prefill":           # the last 200 tokens of the sequence as one chunk
        new = 200
        qkv = rnd(new, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=22)
        q_last = qkv[new - 1, :nh * hd]
    else:
        q = rnd(1, nh * hd, dtype=torch.bfloat16, seed=22)
        q_last = q[0]
    for key_pos, gain in ((first_key - 1, 40.0), (first_key, 30.0)):
        blk = cache.table_host[cache.slots[0], key_pos // 64]
        for kvh in range(nkv):
            own = q_last[kvh * 2 * hd:kvh * 2 * hd + hd].float()     # the group's first head
            cache.k[blk, kvh, key_pos % 64, :] = (own * gain).to(torch.bfloat16)
    if kernel == "prefill":
        out = torch.zeros(new, nh * hd, device=DEV, dtype=torch.bfloat16)
        cu = torch.tensor([0, new], dtype=torch.int32, device=DEV)
        start = torch.tensor([n - new], dtype=torch.int32, device=DEV)
        ops.attn_prefill(qkv, out, cache.k, cache.v, cache.table, cu, start, seq_slot, nh, nkv,
                         hd, 1.0, window, 64, 1, new, fault)
        got = out[new - 1]
    else:
        out = torch.empty(1, nh * hd, device=DEV, dtype=torch.bfloat16)
        tpos = torch.tensor([pos], dtype=torch.int32, device=DEV)
        seq = torch.zeros(1, dtype=torch.int32, device=DEV)
        if kernel == "simt":
            ops.attn_simt(q, out, cache.k, cache.v, cache.table, tpos, seq, seq_slot, nh, nkv,
                          hd, 1.0, window, 64)
        else:
            ops.decode_attention_simt_only(kernel == "decode_cuda_cores")
            try:
                ops.attn_decode(q, out, cache.k, cache.v, cache.table, tpos, seq, seq_slot, nh,
                                nkv, hd, 1.0, window, 64, splits, fault,
                                kernel == "decode_cluster" and splits <= ops.CLUSTER_MAX_RANGES)
            finally:
                ops.decode_attention_simt_only(False)
        got = out[0]
    torch.cuda.synchronize()
    assert fault.item() == 0
    blk = cache.table_host[cache.slots[0], first_key // 64]
    hidden = cache.table_host[cache.slots[0], (first_key - 1) // 64]
    for h in (0, 2):       # the heads whose own query was copied into the keys
        want = cache.v[blk, h // 2, first_key % 64, :]
        close(got[h * hd:(h + 1) * hd], want, 2e-2)
        wrong = cache.v[hidden, h // 2, (first_key - 1) % 64, :]
        assert (got[h * hd:(h + 1) * hd].float() - wrong.float()).abs().max() > 0.5


# ------------------------------------------------------------------ rotary + cache write
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing", [0, 1])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (3, 1, 48, 32), (2, 2, 64, 0)])
def test_rope_kv_append(ops, dtype, pairing, nh, nkv, hd, rot):
    lens = [5, 70]
    cache = ToyCache(lens, nkv, hd, dtype, seed=3)
    k_before, v_before = cache.k.clone(), cache.v.clone()
    theta, P = 10000.0, 128
    half = max(rot // 2, 1)
    j = torch.arange(half, dtype=torch.float64)
    ang = torch.arange(P, dtype=torch.float64)[:, None] / theta ** (2 * j / max(rot, 1))[None, :]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    qpos = [3, 4, 64, 65, 69]
    qseq = [0, 0, 1, 1, 1]
    T = len(qpos)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=8)
    orig = qkv.clone()
    fault = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_kv_append(qkv, cos, sin, pairing, rot, nh, nkv, hd,
                       torch.tensor(qpos, dtype=torch.int32, device=DEV),
                       torch.tensor(qseq, dtype=torch.int32, device=DEV), cache.seq_slot,
                       cache.table, cache.k, cache.v, 64, True, fault)
    assert fault.item() == 0
    tol = 1e-6 if dtype == torch.float32 else 5e-3

    def rotate(x, p):        # x [heads, hd] float64
        y = x.clone()
        for jj in range(rot // 2):
            i0, i1 = (2 * jj, 2 * jj + 1) if pairing else (jj, jj + rot // 2)
            c, s = math.cos(ang[p, jj]), math.sin(ang[p, jj])
            y[:, i0] = x[:, i0] * c - x[:, i1] * s
            y[:, i1] = x[:, i0] * s + x[:, i1] * c
        return y
    touched = set()
    for t in range(T):
        row = orig[t].double().cpu()
        q = row[:nh * hd].reshape(nh, hd)
        k = row[nh * hd:(nh + nkv) * hd].reshape(nkv, hd)
        v = row[(nh + nkv) * hd:].reshape(nkv, hd)
        close(qkv[t, :nh * hd].reshape(nh, hd), rotate(q, qpos[t]), tol)
        blk = cache.table_host[cache.slots[qseq[t]], qpos[t] // 64]
        close(cache.k[blk, :, qpos[t] % 64, :], rotate(k, qpos[t]), tol)
        close(cache.v[blk, :, qpos[t] % 64, :], v, tol)
        touched.add((int(blk), qpos[t] % 64))
    # nothing else in the cache moved
    mask = torch.ones_like(cache.k, dtype=torch.bool)
    for blk, off in touched:
        mask[blk, :, off, :] = False
    assert torch.equal(cache.k[mask], k_before[mask]) and torch.equal(cache.v[mask], v_before[mask])


# ------------------------------------------------------------------ sampling
def test_sample_greedy_ties_lowest(ops):
    V = 1000
    logits = rnd(4, V)
    logits[0, 17] = logits[0, 900] = 50.0
    logits[1, 999] = 60.0
    logits[2, :] = 1.0
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, 0.0, 0, 42)
    want = [17, 999, 0, int(torch.argmax(logits[3]))]
    assert out.tolist() == want


def test_sample_temperature_statistics_and_determinism(ops):
    V, rows = 16, 4096
    base = torch.tensor([float(i % 5) for i in range(V)])
    logits = base[None, :].repeat(rows, 1).to(DEV).contiguous()
    req = torch.arange(rows, dtype=torch.int64, device=DEV)
    draw = torch.zeros(rows, dtype=torch.int32, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, 0.8, 0, 7, req, draw)
    assert draw.min().item() == 1 and draw.max().item() == 1
    freq = torch.bincount(out.long().cpu(), minlength=V).double() / rows
    want = torch.softmax(base.double() / 0.8, dim=0)
    assert (freq - want).abs().max().item() < 0.03
    # same (seed, request, draw) → same token, whatever the batch
    out2 = torch.empty(1, dtype=torch.int32, device=DEV)
    for r in (0, 5, 4000):
        ops.sample(logits[r:r + 1], out2, 0.8, 0, 7, req[r:r + 1],
                   torch.zeros(1, dtype=torch.int32, device=DEV))
        assert out2.item() == out[r].item()
    # another draw number changes the stream
    draw1 = torch.ones(rows, dtype=torch.int32, device=DEV)
    out3 = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, out3, 0.8, 0, 7, req, draw1)
    assert (out3 != out).float().mean().item() > 0.3


def test_sample_top_k(ops):
    V, rows, k = 5000, 2048, 5
    row = rnd(V, scale=2.0).cpu()
    logits = row[None, :].repeat(rows, 1).to(DEV).contiguous()
    req = torch.arange(rows, dtype=torch.int64, device=DEV)
    draw = torch.zeros(rows, dtype=torch.int32, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, 1.3, k, 3, req, draw)
    vals, idx = torch.topk(row, k)
    assert set(out.tolist()) <= set(idx.tolist())
    want = torch.softmax(vals.double() / 1.3, dim=0)
    freq = torch.tensor([(out.cpu() == i).double().mean() for i in idx])
    assert (freq - want).abs().max().item() < 0.04
    # k = 1 is arg-max; a tiny temperature is arg-max
    ops.sample(logits, out, 1.0, 1, 3, req, draw)
    assert set(out.tolist()) == {int(idx[0])}
    ops.sample(logits, out, 1e-4, 0, 3, req, draw)
    assert set(out.tolist()) == {int(idx[0])}
    # the host mirror of the generator agrees with the walk along the sorted candidates
    u = ops.uniform01(3, 11, 0)
    d0 = torch.zeros(1, dtype=torch.int32, device=DEV)
    o1 = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.sample(logits[:1], o1, 1.3, k, 3, torch.tensor([11], dtype=torch.int64, device=DEV), d0)
    cum = torch.cumsum(want, 0)
    pick = int(idx[int((cum >= u).nonzero()[0])]) if (cum >= u).any() else int(idx[-1])
    assert o1.item() == pick
