"""Each kernel alone against its plain PyTorch statement (tests/plain_ops.py), at sizes
other than the engine's: widths that are no power of two, tails, empty groups, one row."""
import math

import pytest
import torch

from plain_ops import PlainOps

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from dlm_b200.ops import native_ops
    return native_ops(fast=True)


@pytest.fixture(scope="module")
def slow_ops():
    from dlm_b200.ops import native_ops
    return native_ops(fast=False)


@pytest.fixture(scope="module")
def ref():
    return PlainOps()


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dtype)


def tol(dtype, k=1):
    # 32-bit: summation order only.  bfloat16: inputs are the same bfloat16 numbers on both sides and sums are
    # 32-bit, so only a bfloat16 output's last rounding differs (one step, 2^-8 relative).
    return dict(rtol=2e-5, atol=2e-5 * math.sqrt(k)) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)


def close(a, b, **kw):
    torch.testing.assert_close(a.float(), b.float(), **kw)


# --------------------------------------------------------------------------- basic
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(ops, ref, dtype):
    table = rand((301, 72), dtype, 0)
    tokens = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device="cuda")
    close(ops.embed(tokens, table), ref.embed(tokens, table), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [72, 2048, 3584, 5000])
def test_rmsnorm(ops, ref, dtype, H):
    x = rand((5, H), torch.float32, 1, 3.0)
    w = 1 + rand((H,), torch.float32, 2, 0.1)
    close(ops.rmsnorm(x, w, 1e-5, dtype), ref.rmsnorm(x, w, 1e-5, dtype), **tol(dtype))
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device="cuda")
    close(ops.rmsnorm(x, w, 3e-6, dtype, rows), ref.rmsnorm(x, w, 3e-6, dtype, rows), **tol(dtype))


@pytest.mark.parametrize("H", [72, 1000, 2048])
def test_rmsnorm_row_does_not_depend_on_the_batch(ops, H):
    # few rows take the kernel with a block per row, many rows the one with a warp per row: same bits
    x = rand((1500, H), torch.float32, 7, 2.0)
    w = 1 + rand((H,), torch.float32, 8, 0.1)
    many = ops.rmsnorm(x, w, 1e-6, torch.float32)
    few = ops.rmsnorm(x[:6].contiguous(), w, 1e-6, torch.float32)
    assert torch.equal(many[:6], few)


def test_rmsnorm_hand_value(ops):
    # src/forward/cpu.rs:1289-1293: rmsnorm([3, 4], eps = 0) = [0.848528, 1.131371]
    x = torch.tensor([[3.0, 4.0]], device="cuda")
    out = ops.rmsnorm(x, torch.ones(2, device="cuda"), 0.0, torch.float32)
    close(out, torch.tensor([[0.848528, 1.131371]], device="cuda"), rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------------ products
GEMM_SHAPES = [(1, 64, 64), (5, 97, 130), (64, 128, 256), (130, 200, 72), (257, 330, 1000), (3, 1408, 2048),
               (8, 2048, 1408), (16, 100, 72), (33, 200, 200), (2, 48, 40), (9, 2816, 2048), (1, 300, 5632),
               (65, 128, 64), (300, 264, 40), (513, 2816, 2048), (1000, 96, 1408), (100, 384, 192),
               # the wider model's shapes: K = 3584 (q|k|v of 28 + 2 * 4 heads), the shared expert's gate/up
               # (N = 2 * 20480) and down (K = 20480) products
               (8, 4608, 3584), (300, 4608, 3584), (4, 40960, 3584), (200, 3584, 20480), (3, 3584, 20480)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_linear(ops, ref, dtype, M, N, K):
    a, w = rand((M, K), dtype, 3), rand((N, K), dtype, 4, 0.05)
    bias = rand((N,), torch.float32, 5)
    close(ops.linear(a, w, bias, torch.float32), ref.linear(a, w, bias, torch.float32), **tol(torch.float32, K))
    close(ops.linear(a, w, None, dtype), ref.linear(a, w, None, dtype), **tol(dtype, K))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_linear_add_and_swiglu(ops, ref, dtype, M, N, K):
    a, w = rand((M, K), dtype, 6), rand((N, K), dtype, 7, 0.05)
    r1 = rand((M, N), torch.float32, 8)
    r2 = r1.clone()
    ops.linear_add(a, w, r1)
    ref.linear_add(a, w, r2)
    close(r1, r2, **tol(torch.float32, K))
    if N % 2 == 0:
        close(ops.linear_swiglu(a, w), ref.linear_swiglu(a, w), **tol(dtype, K))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,k,T,H,I", [(5, 1, 9, 72, 40), (8, 2, 33, 64, 32), (12, 3, 130, 256, 48),
                                       (60, 4, 7, 512, 176), (12, 3, 20, 256, 48), (60, 4, 64, 2048, 1408),
                                       (8, 2, 700, 64, 32), (60, 4, 2048, 512, 176),
                                       (64, 8, 8, 3584, 2560), (64, 8, 300, 3584, 2560)])
def test_grouped_products(ops, ref, dtype, E, k, T, H, I):
    h = rand((T, H), dtype, 9)
    g = torch.Generator().manual_seed(E)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    offsets, rows, dest = ops.moe_permute(ids, E)
    o2, r2, d2 = ref.moe_permute(ids, E)
    assert torch.equal(offsets, o2)
    # order inside a group is free: compare as sets per group, and dest must invert rows
    off = offsets.tolist()
    for e in range(E):
        assert sorted(rows[off[e]:off[e + 1]].tolist()) == sorted(r2[off[e]:off[e + 1]].tolist())
    flat_dest = dest.reshape(-1).long()
    assert sorted(flat_dest.tolist()) == list(range(T * k))
    assert torch.equal(rows[flat_dest].long(), torch.arange(T * k, device="cuda") // k)
    w_gu = rand((E, 2 * I, H), dtype, 10, 0.05)
    w_d = rand((E, H, I), dtype, 11, 0.05)
    act = ops.grouped_swiglu(h, w_gu, offsets, rows)
    close(act, ref.grouped_swiglu(h, w_gu, offsets, rows), **tol(dtype, H))
    y = ops.grouped_linear(act, w_d, offsets)
    close(y, ref.grouped_linear(act, w_d, offsets), **tol(torch.float32, I))
    wts = torch.rand((T, k), device="cuda")
    shared, gate = rand((T, H), torch.float32, 12), torch.rand((T,), device="cuda")
    r1 = rand((T, H), torch.float32, 13)
    r2_ = r1.clone()
    ops.moe_combine(y, dest, wts, shared, gate, r1)
    ref.moe_combine(y, dest, wts, shared, gate, r2_)
    close(r1, r2_, **tol(torch.float32, k))
    r3, r4 = r1.clone(), r1.clone()
    ops.moe_combine(y, dest, wts, None, None, r3)
    ref.moe_combine(y, dest, wts, None, None, r4)
    close(r3, r4, **tol(torch.float32, k))


# -------------------------------------------------------------------------- router
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,k,H,norm,gate", [(5, 1, 72, True, False), (8, 2, 64, False, True),
                                             (12, 3, 256, True, True), (60, 4, 2048, False, True),
                                             (64, 8, 3584, False, True), (130, 6, 100, True, False)])
def test_router(ops, ref, dtype, E, k, H, norm, gate):
    T = 19
    h = rand((T, H), dtype, 14)
    w = rand((E + int(gate), H), dtype, 15, 0.3)
    ids, wts, g = ops.router_topk(h, w, E, k, norm, gate)
    ids2, wts2, g2 = ref.router_topk(h, w, E, k, norm, gate)
    assert torch.equal(ids, ids2)
    close(wts, wts2, rtol=1e-4, atol=1e-6)
    if gate:
        close(g, g2, rtol=1e-4, atol=1e-6)
    # fused form: the 32-bit residual and the norm's weight go in, the norm runs inside
    x = rand((T, H), torch.float32, 16, 2.0)
    nw = 1 + rand((H,), torch.float32, 17, 0.1)
    a = ops.router_topk(x, w, E, k, norm, gate, norm_weight=nw, eps=1e-6)
    b = ref.router_topk(x, w, E, k, norm, gate, norm_weight=nw, eps=1e-6)
    assert torch.equal(a[0], b[0])
    close(a[1], b[1], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,k,H,norm,score,scale,bias", [
    (8, 2, 64, True, "sigmoid", 1.5, True), (12, 3, 256, False, "sigmoid", 1.0, False),
    (60, 4, 2048, True, "softmax", 2.5, True), (130, 6, 100, False, "softmax", 0.5, True)])
def test_router_score_functions(ops, ref, dtype, E, k, H, norm, score, scale, bias):
    """Sigmoid scores, a selection bias that moves the choice but not the weights, a scale factor; and the
    input given as 32-bit activations that are already normalised (weights in the other dtype)."""
    T = 23
    x32 = rand((T, H), torch.float32, 24)
    w = rand((E, H), dtype, 25, 0.3)
    b = rand((E,), torch.float32, 26, 0.2) if bias else None
    got = ops.router_topk(x32, w, E, k, norm, False, score=score, scale=scale, select_bias=b)
    want = ref.router_topk(x32, w, E, k, norm, False, score=score, scale=scale, select_bias=b)
    assert torch.equal(got[0], want[0])
    close(got[1], want[1], rtol=1e-4, atol=1e-6)
    if bias:        # the bias changed some choices, or the case shows nothing
        plain = ref.router_topk(x32, w, E, k, norm, False, score=score, scale=scale)
        assert not torch.equal(plain[0], want[0])


@pytest.mark.parametrize("T", [1, 8, 16, 17, 37, 48, 49, 64, 700])
@pytest.mark.parametrize("E,k,H,gate", [(60, 4, 2048, True), (12, 3, 256, False), (64, 8, 3584, True), (5, 1, 72, False),
                                        (130, 6, 100, False)])
def test_route_in_one_launch_equals_the_separate_kernels(ops, T, E, k, H, gate):
    """Logits, choice and grouping together (one launch up to 48 tokens, of two kinds) give what the separate kernels give,
    bit for bit, also when called again and again (the launch counts its blocks in a global counter)."""
    x = rand((T, H), torch.float32, 27, 2.0)
    nw = 1 + rand((H,), torch.float32, 28, 0.1)
    w = rand((E + int(gate), H), torch.bfloat16, 29, 0.3)
    ids, wts, g = ops.router_topk(x, w, E, k, True, gate, norm_weight=nw, eps=1e-6)
    off, rows, dest = ops.moe_permute(ids, E)
    for settled in (False, True, True):      # settled: the logits are worked out before the dependency wait
        i2, w2, g2, off2, rows2, dest2 = ops.route(x, w, E, k, True, gate, norm_weight=nw, eps=1e-6,
                                                   input_settled=settled)
        assert torch.equal(ids, i2) and torch.equal(wts, w2) and torch.equal(off, off2)
        if gate:
            assert torch.equal(g, g2)
        o = off2.tolist()
        for e in range(E):
            assert sorted(rows2[o[e]:o[e + 1]].tolist()) == sorted(rows[o[e]:o[e + 1]].tolist())
        flat = dest2.reshape(-1).long()
        assert sorted(flat.tolist()) == list(range(T * k))
        assert torch.equal(rows2[flat].long(), torch.arange(T * k, device="cuda") // k)
    ops.check_errors()


def test_router_hand_values_and_ties(ops):
    # src/forward/cpu.rs:1580-1595: logits [1, 2, 0], top-2 -> experts [1, 0]; renormalised weights sum to 1
    h = torch.eye(3, device="cuda")[:1]                     # picks column 0 of w^T
    w = torch.tensor([[1.0, 0, 0], [2.0, 0, 0], [0.0, 0, 0]], device="cuda")
    ids, wts, _ = ops.router_topk(h, w, 3, 2, True, False)
    assert ids.tolist() == [[1, 0]]
    assert abs(float(wts.sum()) - 1) < 1e-6
    ids2, wts2, _ = ops.router_topk(h, w, 3, 2, False, False)
    assert abs(float(wts2[0, 0] / wts2[0, 1]) - float(wts[0, 0] / wts[0, 1])) < 1e-5
    # src/forward/cpu.rs:1649-1689: equal logits -> equal halves; ties go to the lower index
    w0 = torch.zeros((4, 3), device="cuda")
    ids3, wts3, _ = ops.router_topk(h, w0, 4, 2, True, False)
    assert ids3.tolist() == [[0, 1]] and wts3.tolist() == [[0.5, 0.5]]


# ------------------------------------------------------------------ rotary + cache
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rd", [(4, 2, 16, 16), (3, 1, 48, 48), (8, 4, 32, 16), (2, 2, 128, 128)])
def test_rope_kv_write(ops, ref, dtype, nh, nkv, hd, rd):
    from dlm_b200.parts.rope import rope_inv_freqs
    T, ps, pages = 11, 16, 6
    qkv = rand((T, (nh + 2 * nkv) * hd), torch.float32, 16)
    pos = torch.tensor([0, 1, 2, 50, 51, 1000, 4095, 7, 8, 9, 10], dtype=torch.int32, device="cuda")
    slots = torch.tensor([0, 1, 17, 95, 80, 33, 34, 35, -1, 64, 15], dtype=torch.int32, device="cuda")
    inv = rope_inv_freqs(hd, 10000.0, rd).cuda()
    k1 = torch.zeros((pages, nkv, ps, hd), dtype=dtype, device="cuda")
    v1, k2, v2 = k1.clone(), k1.clone(), k1.clone()
    q1 = ops.rope_kv_write(qkv, pos, inv, rd, slots, k1, v1, nh, nkv, hd, dtype)
    q2 = ref.rope_kv_write(qkv, pos, inv, rd, slots, k2, v2, nh, nkv, hd, dtype)
    t = dict(rtol=1e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    close(q1, q2, **t)
    close(k1, k2, **t)
    close(v1, v2, rtol=0, atol=0)
    # no rotation, no write
    k3 = torch.zeros_like(k1)
    q3 = ops.rope_kv_write(qkv, pos, None, 0, None, k3, k3.clone(), nh, nkv, hd, dtype)
    close(q3, qkv[:, :nh * hd].to(dtype), rtol=0, atol=0)
    assert float(k3.abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rd", [(4, 2, 16, 16), (3, 1, 48, 24), (2, 2, 128, 128)])
def test_rope_interleaved_pairs(ops, ref, dtype, nh, nkv, hd, rd):
    from dlm_b200.parts.rope import rope_inv_freqs
    T, ps, pages = 7, 16, 3
    qkv = rand((T, (nh + 2 * nkv) * hd), torch.float32, 18)
    pos = torch.tensor([0, 1, 2, 50, 1000, 4095, 7], dtype=torch.int32, device="cuda")
    slots = torch.tensor([0, 1, 17, 40, 33, -1, 15], dtype=torch.int32, device="cuda")
    inv = rope_inv_freqs(hd, 10000.0, rd).cuda()
    k1 = torch.zeros((pages, nkv, ps, hd), dtype=dtype, device="cuda")
    v1, k2, v2 = k1.clone(), k1.clone(), k1.clone()
    q1 = ops.rope_kv_write(qkv, pos, inv, rd, slots, k1, v1, nh, nkv, hd, dtype, interleaved=True)
    q2 = ref.rope_kv_write(qkv, pos, inv, rd, slots, k2, v2, nh, nkv, hd, dtype, interleaved=True)
    t = dict(rtol=1e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    close(q1, q2, **t)
    close(k1, k2, **t)
    close(v1, v2, rtol=0, atol=0)
    # and it is another rotation than the split-half one
    q3 = ref.rope_kv_write(qkv, pos, inv, rd, None, k2, v2, nh, nkv, hd, dtype)
    assert float((q3.float() - q2.float()).abs().max()) > 0.1


def test_rope_identity_at_zero_and_norm(ops):
    # src/forward/cpu.rs:1296-1322: identity at position 0, norms preserved
    from dlm_b200.parts.rope import rope_inv_freqs
    nh, nkv, hd = 2, 1, 8
    inv = rope_inv_freqs(hd, 10000.0).cuda()
    close(inv.cpu(), torch.tensor([1.0, 1e4 ** -0.25, 1e4 ** -0.5, 1e4 ** -0.75]), rtol=1e-6, atol=1e-6)
    qkv = rand((2, (nh + 2 * nkv) * hd), torch.float32, 17)
    pos = torch.tensor([0, 9], dtype=torch.int32, device="cuda")
    k = torch.zeros((1, nkv, 16, hd), device="cuda")
    q = ops.rope_kv_write(qkv, pos, inv, hd, None, k, k.clone(), nh, nkv, hd, torch.float32)
    close(q[0], qkv[0, :nh * hd], rtol=0, atol=0)
    close(q[1].view(nh, hd).norm(dim=-1), qkv[1, :nh * hd].view(nh, hd).norm(dim=-1), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("E,H,I,counts", [
    (6, 2048 + 512, 96, [40, 0, 1, 0, 3, 2]),      # one expert far above the mean: several passes over its rows
    (4, 5632, 64, [0, 17, 0, 5]),                  # rows longer than one stage: chunks of K
    (3, 264, 1408, [9, 9, 9]),
    # at most 1.125 rows per expert on average (the weight-streaming kernel's share), one expert with
    # many: its rows go in passes of 8; rows of two chunks (held in registers) and of three (fetched per chunk)
    (40, 2560, 96, [30] + [0] * 30 + [1] * 9),
    (40, 5632, 64, [0] * 20 + [21] + [1] * 19),
    (40, 1408, 264, [2, 0, 0, 19] + [1] * 20 + [0] * 16),
])
def test_grouped_products_skewed(ops, ref, E, H, I, counts):
    """Rows very unevenly spread over the experts, experts without rows among them, on both grouped kernels (the
    tcgen05 kernel from 1.125 rows per expert on average, the weight-streaming kernel below)."""
    dtype = torch.bfloat16
    M = sum(counts)
    offsets = torch.tensor([0] + torch.tensor(counts).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(5)
    T = 23
    h = rand((T, H), dtype, 14)
    rows = torch.randint(0, T, (M,), generator=g).to(torch.int32).cuda()
    w_gu = rand((E, 2 * I, H), dtype, 15, 0.05)
    w_d = rand((E, H, I), dtype, 16, 0.05)
    act = ops.grouped_swiglu(h, w_gu, offsets, rows)
    close(act, ref.grouped_swiglu(h, w_gu, offsets, rows), **tol(dtype, H))
    y = ops.grouped_linear(act, w_d, offsets)
    close(y, ref.grouped_linear(act, w_d, offsets), **tol(torch.float32, I))
    ops.check_errors()


# ----------------------------------------------------------------------- attention
def build_paged(reqs, nkv, hd, ps, dtype, seed, shuffle=True):
    """reqs: list of (kv_len, q_len).  Returns q, caches, table, cu_q, kv_len with pages scattered."""
    total_pages = sum(-(-n // ps) for n, _ in reqs) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total_pages, generator=g).tolist() if shuffle else list(range(total_pages))
    k = rand((total_pages, nkv, ps, hd), dtype, seed + 1)
    v = rand((total_pages, nkv, ps, hd), dtype, seed + 2)
    width = max(-(-n // ps) for n, _ in reqs) + 1
    table = torch.full((len(reqs), width), -1, dtype=torch.int32)
    cu, it = [0], iter(perm)
    for r, (n, ql) in enumerate(reqs):
        for i in range(-(-n // ps)):
            table[r, i] = next(it)
        cu.append(cu[-1] + ql)
    return (k, v, table.cuda(), torch.tensor(cu, dtype=torch.int32, device="cuda"),
            torch.tensor([n for n, _ in reqs], dtype=torch.int32, device="cuda"))


ATT_CASES = [
    # nh, nkv, hd, page, window, [(kv_len, q_len)]
    (4, 2, 16, 16, 0, [(1, 1), (33, 33), (70, 1), (40, 7)]),
    (3, 1, 48, 16, 24, [(100, 100), (64, 1), (65, 2), (24, 24), (25, 1)]),
    (8, 4, 32, 64, 16, [(200, 17), (16, 16), (17, 17), (129, 1)]),
    (16, 16, 128, 64, 0, [(300, 40), (1024, 1), (65, 65)]),
    (14, 2, 128, 32, 0, [(257, 1), (90, 90)]),
    (4, 2, 128, 64, 0, [(700, 700), (130, 2), (64, 64), (391, 129)]),
    (2, 2, 128, 64, 100, [(600, 600), (300, 37), (1000, 255)]),
    (3, 1, 128, 128, 0, [(513, 513), (129, 128)]),
    (2, 1, 256, 16, 0, [(50, 50), (33, 1)]),
    (4, 4, 80, 16, 40, [(130, 130)]),
    # single tokens only: lengths around a tile's and a page's edge, more heads in a group than a tile has rows
    (20, 1, 64, 128, 0, [(1, 1), (63, 1), (64, 1), (65, 1), (1500, 1), (128, 1), (129, 1)]),
    (4, 2, 128, 256, 200, [(700, 1), (199, 1), (200, 1), (201, 1), (5000, 1), (257, 1)]),
    (6, 3, 64, 64, 0, [(4097, 1), (17, 1)]),
    # 7 query heads to a kv head (28 / 4), prompt portions and single tokens
    (28, 4, 128, 64, 0, [(300, 300), (700, 1), (2500, 130)]),
    (28, 4, 128, 64, 0, [(3000, 1), (64, 1), (1, 1)]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps,window,reqs", ATT_CASES)
@pytest.mark.parametrize("fast", [False, True])
def test_attention(ops, slow_ops, ref, dtype, nh, nkv, hd, ps, window, reqs, fast):
    o = ops if fast else slow_ops
    k, v, table, cu_q, kv_len = build_paged(reqs, nkv, hd, ps, dtype, 21)
    if window:
        # pages a window has passed are not there any more
        for r, (n, ql) in enumerate(reqs):
            lo = max(0, n - ql - window + 1)
            table[r, :lo // ps] = -1
    T = int(cu_q[-1])
    q = rand((T, nh * hd), dtype, 22)
    scale = 1 / math.sqrt(hd)
    mq, mk = max(q for _, q in reqs), max(n for n, _ in reqs)
    ns = sum(1 for _, ql in reqs if ql == 1)
    got = o.attention(q, k, v, table, cu_q, kv_len, window, scale, nh, nkv, hd, mq, mk, ns)
    want = ref.attention(q, k, v, table, cu_q, kv_len, window, scale, nh, nkv, hd, mq, mk)
    close(got, want, **(dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-2)))
    o.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fast", [False, True])
@pytest.mark.parametrize("far", [0, 3, 63, 64, 500, 698])
def test_attention_far_key_stands_out(ops, slow_ops, dtype, fast, far):
    """One key among 700 gets a score far above the rest: the output must be that key's value
    (a kernel that drops a page, a tile or the first/last key cannot pass)."""
    o = ops if fast else slow_ops
    nh, nkv, hd, ps, n = 4, 2, 64, 64, 700
    k, v, table, cu_q, kv_len = build_paged([(n, 1)], nkv, hd, ps, dtype, 31)
    q = rand((1, nh * hd), dtype, 32)
    page, off = int(table[0, far // ps]), far % ps
    for h in range(nkv):
        k[page, h, off] = (q[0, (h * (nh // nkv)) * hd:(h * (nh // nkv) + 1) * hd].float() * 40).to(dtype)
    # every query head of the group must see it: give all heads of a group the same query
    for h in range(nh):
        g = h // (nh // nkv)
        q[0, h * hd:(h + 1) * hd] = q[0, (g * (nh // nkv)) * hd:(g * (nh // nkv) + 1) * hd]
    got = o.attention(q, k, v, table, cu_q, kv_len, 0, 1 / math.sqrt(hd), nh, nkv, hd, 1, n, 1).float().view(nh, hd)
    for h in range(nh):
        close(got[h], v[page, h // (nh // nkv), off].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("fast", [False, True])
def test_attention_window_edge(ops, slow_ops, fast):
    """The key at p - W + 1 is the last one seen, the key at p - W is not."""
    o = ops if fast else slow_ops
    nh = nkv = 1
    hd, ps, W, n = 32, 16, 20, 90
    dtype = torch.float32
    k, v, table, cu_q, kv_len = build_paged([(n, 1)], nkv, hd, ps, dtype, 41, shuffle=False)
    q = rand((1, hd), dtype, 42)
    p = n - 1
    for j, boost in ((p - W + 1, 30.0), (p - W, 60.0)):
        k[j // ps, 0, j % ps] = q[0] * boost
    got = o.attention(q, k, v, table, cu_q, kv_len, W, 1 / math.sqrt(hd), nh, nkv, hd, 1, n, 1)
    inside = p - W + 1
    close(got[0], v[inside // ps, 0, inside % ps], rtol=1e-3, atol=1e-3)


# ------------------------------------------------------------------------ sampling
def test_argmax_first_maximum(ops, ref):
    lg = rand((6, 1000), torch.float32, 51)
    lg[0, 17] = lg[0, 900] = 50.0          # src/generate.rs:518-521: the first maximum wins
    lg[1, :] = 1.0
    lg[2, 999] = 99.0
    assert ops.argmax(lg).tolist() == ref.argmax(lg).tolist()
    assert ops.argmax(lg)[:3].tolist() == [17, 0, 999]
    big = rand((3, 151936), torch.float32, 52)
    assert ops.argmax(big).tolist() == torch.argmax(big, dim=-1).tolist()


@pytest.mark.parametrize("V,reps", [(301, 1), (5000, 1), (151936, 1), (151936, 2), (151936, 4), (40000, 7)])
def test_sampler_against_plain(ops, ref, V, reps):
    """``reps`` repeats the 12 rows: with a large vocabulary a row is shared by 8, 4, 2 or 1 blocks, the fewer the
    more rows the launch has."""
    N = 12
    lg = rand((N, V), torch.float32, 53, 2.0)
    lg[3, 5] = lg[3, 100] = lg[3].max() + 1        # tied best candidates
    params = torch.tensor([[0.8, 1.0, 0.0, 1.0], [1.0, 0.9, 0.0, 1.0], [0.7, 1.0, 0.05, 1.0], [1.0, 1.0, 0.0, 1.0],
                           [0.0, 1.0, 0.0, 1.3], [1.3, 0.5, 0.1, 1.2], [0.8, 1.0, 0.0, 1.0], [0.5, 0.3, 0.0, 1.0],
                           [2.0, 1.0, 0.0, 1.0], [1.0, 0.99, 0.0, 1.0], [0.8, 1.0, 0.9, 1.0], [1.0, 1.0, 0.0, 2.0]],
                          device="cuda")
    top_k = torch.tensor([0, 0, 0, 0, 0, 50, 1, 0, 7, 0, 0, 20], dtype=torch.int32, device="cuda")
    seen_offsets = torch.arange(0, 4 * (N + 1), 4, dtype=torch.int32, device="cuda")
    # spread over the vocabulary, so that with a large one the blocks that share a row penalise each other's parts
    seen_tokens = ((torch.arange(4 * N, dtype=torch.int64, device="cuda") * 37123) % V).to(torch.int32)
    if reps > 1:
        lg, params, top_k = lg.repeat(reps, 1), params.repeat(reps, 1), top_k.repeat(reps)
        seen_offsets = torch.arange(0, 4 * (N * reps + 1), 4, dtype=torch.int32, device="cuda")
        seen_tokens = seen_tokens.repeat(reps)
    agree = total = 0
    for trial in range(6 if reps == 1 else 2):
        u = torch.rand((N * reps,), generator=torch.Generator().manual_seed(trial)).cuda()
        got = ops.sample(lg, params, top_k, u, seen_offsets, seen_tokens)
        want = ref.sample(lg, params, top_k, u, seen_offsets, seen_tokens)
        agree += int((got == want).sum())
        total += N * reps
        assert int(got[6]) == int(torch.argmax(lg[6]))          # top_k = 1 is greedy
    assert agree >= total - reps       # a draw within rounding of a boundary may fall either way


def test_repetition_penalty_hand_values(ops):
    # src/generate.rs:575-577: logits [2, 2, -2, -2], seen {0, 2}... penalty 2 -> [1, 2, -4, -2]; greedy picks 1
    lg = torch.tensor([[2.0, 2.0, -2.0, -2.0]], device="cuda")
    params = torch.tensor([[0.0, 1.0, 0.0, 2.0]], device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.sample(lg, params, z, torch.zeros(1, device="cuda"),
                     torch.tensor([0, 2], dtype=torch.int32, device="cuda"),
                     torch.tensor([0, 2], dtype=torch.int32, device="cuda"))
    assert out.tolist() == [1]
