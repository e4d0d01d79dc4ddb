"""Each part alone against the plain implementation's function for it, at sizes that are
not the tiny models': norm, rotary position encoding, attention, dense and routed
feed-forward, and the block that arranges them."""
import math

import pytest
import torch

import plain_qwen2_moe as plain

pytestmark = pytest.mark.gpu


def runtime(dtype):
    from dlm_b200.engine import make_runtime
    return make_runtime(dtype)


def rnd_of(dtype):
    return plain.bf16_round if dtype == "bfloat16" else (lambda t: t)


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)


class OneLayerCache:
    """The least a mixer needs of a cache: one request, pages 0..n in order."""

    def __init__(self, rt, nkv, hd, tokens, page_size=16, window=0):
        from dlm_b200.parts.base import GroupView, PagedView, StepBatch
        pages = -(-tokens // page_size)
        dev = rt.device
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        self.k = torch.zeros((pages + 1, nkv, page_size, hd), dtype=rt.dtype, device=dev)
        self.v = torch.zeros_like(self.k)
        group = GroupView(slots=i32(list(range(tokens))), block_table=i32([list(range(pages))]),
                          page_size=page_size, window=window)
        self.batch = StepBatch(num_tokens=tokens, num_requests=1, tokens=i32([0] * tokens),
                               positions=i32(list(range(tokens))), token_req=i32([0] * tokens), cu_q=i32([0, tokens]),
                               kv_len=i32([tokens]), state_slot=i32([0]), logit_rows=i32([]), groups=[group],
                               max_q_len=tokens, max_kv_len=tokens, num_single=0)
        self.view = PagedView({"k": self.k, "v": self.v}, group, write=True)

    def context(self, rt):
        from dlm_b200.parts.base import StepContext
        return StepContext(rt, self.batch, lambda call: self.view, lambda call: None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from dlm_b200.parts.norm import RMSNorm
    rt = runtime(dtype)
    part = RMSNorm(200, 3e-6)
    w = 1 + 0.1 * torch.randn(200)
    part.load({"weight": w}, rt)
    x = 2 * torch.randn(7, 200)
    want = rnd_of(dtype)(plain.rmsnorm(x.double(), w.double(), 3e-6))
    torch.testing.assert_close(part.forward(x.cuda(), rt).double().cpu(), want, **tol(dtype))


def test_rotary_part_table():
    from dlm_b200.parts.rope import RotaryNeoX
    rt = runtime("float32")
    pe = RotaryNeoX(48, 50000.0)
    table, rd = pe.rotary(rt)
    assert rd == 48 and torch.equal(table.cpu(), plain.rope_inv_freqs(48, 50000.0))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,window,bias", [(6, 2, 32, None, True), (5, 5, 48, 20, False), (4, 1, 80, 33, True)])
def test_attention_part(dtype, nh, nkv, hd, window, bias):
    from dlm_b200.parts.attention import GroupedQueryAttention
    from dlm_b200.parts.base import PartSpec
    torch.manual_seed(nh)
    rt = runtime(dtype)
    H, T, theta = 136, 90, 30000.0
    part = GroupedQueryAttention(H, nh, nkv, hd, qkv_bias=None, window=window,
                                 position=PartSpec("rope_neox", {"head_dim": hd, "theta": theta}))
    tensors = {f"{n}_proj.weight": 0.05 * torch.randn(d, H) for n, d in (("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd))}
    tensors["o_proj.weight"] = 0.05 * torch.randn(H, nh * hd)
    if bias:
        tensors.update({f"{n}_proj.bias": 0.1 * torch.randn(d) for n, d in (("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd))})
    part.load(tensors, rt)
    rnd = rnd_of(dtype)
    h = rnd(torch.randn(T, H).double())
    # the plain statement, with the same rounding places
    W = {k: (rnd(v.double()) if k.endswith("weight") else v.double()) for k, v in tensors.items()}
    q, k, v = (h @ W[f"{n}_proj.weight"].T + (W[f"{n}_proj.bias"] if bias else 0) for n in "qkv")
    pos, inv = torch.arange(T), plain.rope_inv_freqs(hd, theta)
    q = rnd(plain.rope(q.view(T, nh, hd), pos, inv))
    k = rnd(plain.rope(k.view(T, nkv, hd), pos, inv))
    ctx = rnd(plain.attention(q, k, rnd(v.view(T, nkv, hd)), window).reshape(T, nh * hd))
    want = ctx @ W["o_proj.weight"].T
    cache = OneLayerCache(rt, nkv, hd, T, window=window or 0)
    resid = torch.zeros(T, H, device="cuda")
    part.forward(h.to(rt.dtype).cuda(), resid, cache.context(rt), 0)
    torch.testing.assert_close(resid.double().cpu(), want, **tol(dtype))
    # the keys were stored rotated, the values as projected
    torch.testing.assert_close(cache.k[:-1].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:T].double().cpu(), k, **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dense_ffn_part(dtype):
    from dlm_b200.parts.ffn import DenseSwiGLU
    torch.manual_seed(1)
    rt = runtime(dtype)
    H, I, T = 136, 88, 21
    part = DenseSwiGLU(H, I)
    t = {"gate_proj.weight": 0.1 * torch.randn(I, H), "up_proj.weight": 0.1 * torch.randn(I, H),
         "down_proj.weight": 0.1 * torch.randn(H, I)}
    part.load(t, rt)
    rnd = rnd_of(dtype)
    h = rnd(torch.randn(T, H).double())
    want = plain.swiglu_ffn(h, *(rnd(t[f"{n}_proj.weight"].double()) for n in ("gate", "up", "down")), rnd)
    resid = torch.ones(T, H, device="cuda")
    part.forward(h.to(rt.dtype).cuda(), resid, type("C", (), {"rt": rt})())
    torch.testing.assert_close(resid.double().cpu() - 1, want, **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [37, 9, 1])       # 9 and 1: routing in one launch
@pytest.mark.parametrize("E,k,norm,Is,gate", [(6, 2, True, 40, True), (10, 3, False, None, False), (7, 1, True, 24, False)])
def test_moe_part(dtype, E, k, norm, Is, gate, T):
    from dlm_b200.parts.ffn import SoftmaxTopKMoE
    from dlm_b200.parts.norm import RMSNorm
    torch.manual_seed(E)
    rt = runtime(dtype)
    H, I = 72, 24
    part = SoftmaxTopKMoE(H, E, k, I, norm, shared_intermediate_size=Is, shared_gate=gate)
    t = {"gate.weight": 0.5 * torch.randn(E, H)}
    for e in range(E):
        t.update({f"experts.{e}.gate_proj.weight": 0.1 * torch.randn(I, H), f"experts.{e}.up_proj.weight": 0.1 * torch.randn(I, H),
                  f"experts.{e}.down_proj.weight": 0.1 * torch.randn(H, I)})
    if Is:
        t.update({"shared_expert.gate_proj.weight": 0.1 * torch.randn(Is, H), "shared_expert.up_proj.weight": 0.1 * torch.randn(Is, H),
                  "shared_expert.down_proj.weight": 0.1 * torch.randn(H, Is)})
        if gate:
            t["shared_expert_gate.weight"] = 0.3 * torch.randn(1, H)
    assert sorted(p.name for p in part.param_specs()) == sorted(t)
    part.load(t, rt)
    rnd = rnd_of(dtype)
    norm_part = RMSNorm(H, 1e-6)
    nw = 1 + 0.1 * torch.randn(H)
    norm_part.load({"weight": nw}, rt)
    x = torch.randn(T, H)
    n_full = plain.rmsnorm(x.double(), nw.double(), 1e-6)
    lw = {"router": rnd(t["gate.weight"].double()),
          "experts": [tuple(rnd(t[f"experts.{e}.{n}_proj.weight"].double()) for n in ("gate", "up", "down")) for e in range(E)]}
    if Is:
        lw["shared"] = tuple(rnd(t[f"shared_expert.{n}_proj.weight"].double()) for n in ("gate", "up", "down"))
        if gate:
            lw["shared_gate"] = rnd(t["shared_expert_gate.weight"].double())
    cfg = type("Cfg", (), {"k": k, "E": E, "norm_topk": norm})()
    want = plain.moe_ffn(rnd(n_full), lw, cfg, rnd, x_router=n_full)
    resid = x.clone().cuda()
    ctx = type("C", (), {"rt": rt})()
    part.forward(norm_part.forward(resid, rt), resid, ctx, pre_norm=norm_part)
    torch.testing.assert_close(resid.double().cpu() - x.double(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part_equals_plain_layer(dtype, tiny_folders):
    """The pre-norm block of tiny B's routed, windowed layer 1 against decoder_layer."""
    from dlm_b200.engine import Engine
    eng = Engine.from_pretrained(tiny_folders["B"], dtype=dtype, page_size=16, num_pages=8, max_requests=2)
    oracle = plain.PlainModel(tiny_folders["B"], compute=torch.float64, emulate_bf16=(dtype == "bfloat16"))
    T = 50
    x = torch.randn(T, 256)
    plain.MARGIN_LOG = []
    try:
        want = plain.decoder_layer(x.double(), oracle.layers[1], oracle.cfg, 1, torch.arange(T), oracle.inv_freq,
                                   oracle.rnd)
        margins = plain.MARGIN_LOG[0]
    finally:
        plain.MARGIN_LOG = None
    # rows whose routing is a near-tie for this precision are not compared (see test_engine_gpu.py)
    keep = margins >= (1e-6 if dtype == "float32" else 2e-4)
    assert int(keep.sum()) > T // 2
    s = eng.cache.open()
    eng.cache.append([(s, T)])
    batch = eng.cache.make_batch([(s, [0] * T, [])])
    from dlm_b200.parts.base import StepContext
    ctx = StepContext(eng.rt, batch, lambda call: eng.cache.paged_view(call, batch), eng.cache.state_tensor)
    resid = x.clone().cuda()
    eng.model.blocks[1].forward(resid, ctx, 1)
    torch.testing.assert_close(resid.double().cpu()[keep], want[keep],
                               **(dict(rtol=1e-4, atol=1e-4) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)))
