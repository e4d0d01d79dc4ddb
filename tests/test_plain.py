"""The plain implementation itself: the hand-derivable values the reference asserts in its
own unit tests, restated (src/forward/cpu.rs:1281-1723, src/generate.rs:517-721)."""
import math

import pytest
import torch

import plain_qwen2_moe as P
from tiny_configs import TINY, prompt


def test_rmsnorm_value():
    out = P.rmsnorm(torch.tensor([3.0, 4.0]), torch.ones(2), 0.0)       # cpu.rs:1289-1293
    assert torch.allclose(out, torch.tensor([0.848528, 1.131371]), atol=1e-5)


def test_softmax_and_silu():
    s = P.softmax(torch.tensor([1.0, 2.0, 3.0]))
    assert abs(float(s.sum()) - 1) < 1e-6 and float(P.silu(torch.tensor(0.0))) == 0.0


def test_rope_table_identity_and_norm():
    f = P.rope_inv_freqs(8, 1e4)                                          # cpu.rs:1325-1333
    assert torch.allclose(f, torch.tensor([1.0, 1e4 ** -0.25, 1e4 ** -0.5, 1e4 ** -0.75]), atol=1e-6)
    x = torch.randn(2, 3, 8)
    r = P.rope(x, torch.tensor([0, 5]), f)
    assert torch.equal(r[0], x[0])
    assert torch.allclose(r[1].norm(dim=-1), x[1].norm(dim=-1), atol=1e-5)


def test_route_topk():
    ids, w = P.route_topk(torch.tensor([[1.0, 2.0, 0.0]]), 2, True)       # cpu.rs:1580-1595
    assert ids.tolist() == [[1, 0]] and abs(float(w.sum()) - 1) < 1e-6
    _, w2 = P.route_topk(torch.tensor([[1.0, 2.0, 0.0]]), 2, False)
    assert abs(float(w[0, 0] / w[0, 1]) - float(w2[0, 0] / w2[0, 1])) < 1e-6
    ids3, w3 = P.route_topk(torch.zeros(1, 4), 2, True)                   # cpu.rs:1649-1689; ties: lower index
    assert ids3.tolist() == [[0, 1]] and w3.tolist() == [[0.5, 0.5]]


def test_attention_single_position_and_gqa():
    q = torch.randn(1, 4, 8)
    k, v = torch.randn(1, 2, 8), torch.randn(1, 2, 8)
    out = P.attention(q, k, v, None)                                      # cpu.rs:1372-1444
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 1], v[0, 0])
    assert torch.allclose(out[0, 2], v[0, 1]) and torch.allclose(out[0, 3], v[0, 1])


def test_window_mask():
    T, W = 10, 3
    q = torch.zeros(T, 1, 4)
    k = torch.zeros(T, 1, 4)
    v = torch.arange(T, dtype=torch.float32)[:, None, None].expand(T, 1, 4).clone()
    out = P.attention(q, k, v, W)           # equal scores: the mean of the visible values
    for p in range(T):
        lo = max(0, p - W + 1)
        assert abs(float(out[p, 0, 0]) - (lo + p) / 2) < 1e-6


def test_sampler_values():
    assert P.argmax(torch.tensor([1.0, 3.0, 3.0])) == 1                   # generate.rs:518-521
    pen = P.apply_repetition_penalty(torch.tensor([2.0, 2.0, -2.0, -2.0]), [0, 2], 2.0)
    assert pen.tolist() == [1.0, 2.0, -4.0, -2.0]                         # generate.rs:575-577
    lg = torch.tensor([0.1, 5.0, 0.2, 4.9])
    for seed in range(5):
        assert P.sample_topk_topp(lg, 1.0, 1.0, 1, 0.0, P.SplitMix64(seed)) == 1          # top_k = 1
        assert P.sample_topk_topp(lg, 1.0, 0.05, 0, 0.0, P.SplitMix64(seed)) == 1         # tight nucleus
        assert P.sample_topk_topp(lg, 1.0, 1.0, 0, 0.95, P.SplitMix64(seed)) in (1,)      # min-p keeps the top
    a = [P.sample_topk_topp(lg, 1.0, 1.0, 0, 0.0, P.SplitMix64(3)) for _ in range(3)]
    assert a[0] == a[1] == a[2]                                            # seeded: reproducible
    r = P.SplitMix64(0)
    assert all(0.0 <= r.next_f32() < 1.0 for _ in range(100))


def test_model_invariants(tiny_folders):
    for name in TINY:
        m = P.PlainModel(tiny_folders[name], compute=torch.float64)
        toks = prompt(1, 40, m.cfg.V)
        full = m.logits(toks)
        assert full.shape == (40, m.cfg.V)
        # causal: a prefix gives the same logits
        assert torch.allclose(m.logits(toks[:17]), full[:17], atol=1e-6)
        # an expert no token is routed to cannot change the output (cpu.rs:1598-1646)
        m32 = P.PlainModel(tiny_folders[name], compute=torch.float32)
        assert float((m32.logits(toks) - full).abs().max()) < 1e-4
        bf = P.PlainModel(tiny_folders[name], compute=torch.float64, emulate_bf16=True)
        assert 1e-5 < float((bf.logits(toks) - full).abs().max()) < 0.2


def test_windowed_layers_forget(tiny_folders):
    """Tiny C: every layer is windowed (24) and it has 2 layers, so the logits at a position
    depend on at most the last 2 * 23 + 1 tokens."""
    m = P.PlainModel(tiny_folders["C"], compute=torch.float64)
    V = m.cfg.V
    a = prompt(2, 120, V)
    b = list(a)
    b[10] = (b[10] + 1) % V
    la, lb = m.logits(a), m.logits(b)
    assert float((la[10] - lb[10]).abs().max()) > 1e-6
    assert float((la[10 + 47:] - lb[10 + 47:]).abs().max()) == 0.0


def test_generate_eos_included(tiny_folders):
    m = P.PlainModel(tiny_folders["A"], compute=torch.float32)
    p = prompt(4, 6, m.cfg.V)
    out = P.generate(m, p, 8)
    assert len(out) == 8
    stop = out[3]
    cut = P.generate(m, p, 8, eos_token=stop)
    assert cut == out[:out.index(stop) + 1]                                # generate.rs:364-368
    with pytest.raises(ValueError):
        m.logits([])
    with pytest.raises(ValueError):
        m.logits([m.cfg.V])
