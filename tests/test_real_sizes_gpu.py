"""The engine at the layer sizes of Qwen1.5-MoE-A2.7B (two layers of them, the whole vocabulary, random
weights) and of Qwen2-57B-A14B (one layer: hidden 3584, 28 query heads on 4 kv heads, 64 experts of
which 8 are chosen, a shared expert 20,480 wide) against the plain implementation, in 32-bit and in bfloat16, under every way of cutting the work.
At these sizes the bfloat16 path runs the tcgen05 GEMM and attention, the weight-streaming GEMM and the
tensor-core decode attention, and sums are 2,048 to 5,632 terms long.  The plain implementation is the one
of the other tests (double precision, whole sequences, no cache); it computes on the GPU here only because
the CPU would take minutes for the same PyTorch statements."""
import pytest
import torch

import cuttings
import plain_qwen2_moe as plain

pytestmark = pytest.mark.gpu

SIZES = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=2, hidden_size=2048, num_attention_heads=16, num_key_value_heads=16,
    num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
    norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=5632,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, use_sliding_window=False,
    tie_word_embeddings=False, qkv_bias=True)
SIZES_WIDE = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=1, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
    num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
    norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=18944,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, use_sliding_window=False,
    tie_word_embeddings=False, qkv_bias=True)
TOL_F32 = 1e-4
MARGIN_F32 = 1e-6                                   # see test_engine_gpu.py
FLOOR_BF16 = 0.3        # share of positions that must be comparable in bfloat16 (set just under what is seen)


def build(dtype, sizes=SIZES):
    from dlm_b200.config import Qwen2MoeConfig
    from dlm_b200.engine import Engine
    from dlm_b200.weights.random_init import random_state_dict
    cfg = Qwen2MoeConfig.from_dict(sizes)
    eng = Engine.from_random(cfg, seed=5, dtype=dtype, page_size=64, num_pages=16, max_requests=4,
                             max_step_tokens=1024, max_context=1024)
    tensors = random_state_dict(eng.model.param_specs(), 5, torch.float32, "cuda")
    g = torch.Generator().manual_seed(9)
    reqs = {f"r{i}": torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate([300, 40, 150, 9])}
    return cfg, eng, tensors, reqs


def cuttings_of(reqs):
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=3)
    return cuttings.whole(reqs), cuttings.tail_decode(reqs, 32), cuttings.portions(reqs), mixed


@pytest.mark.parametrize("sizes", [SIZES, SIZES_WIDE], ids=["a2.7b", "57b"])
def test_real_layer_sizes_float32(sizes):
    cfg, eng, tensors, reqs = build("float32", sizes)
    oracle = plain.PlainModel((cfg.to_dict(), tensors), compute=torch.float64, device="cuda")
    del tensors
    ref = {rid: oracle.logits(t) for rid, t in reqs.items()}
    margins = {rid: oracle.router_margins(t) for rid, t in reqs.items()}
    compared = total = 0
    for steps in cuttings_of(reqs):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(map(len, reqs.values()))
        for (rid, p), row in got.items():
            total += 1
            if float(margins[rid][p]) < MARGIN_F32:
                continue
            d = float((row - ref[rid][p]).abs().max())
            assert d <= TOL_F32, f"{rid} position {p}: max abs diff {d:.3e}"
            compared += 1
    print(f"compared {compared} of {total} positions")
    assert compared >= 0.9 * total


@pytest.mark.parametrize("sizes", [SIZES, SIZES_WIDE], ids=["a2.7b", "57b"])
def test_real_layer_sizes_bfloat16(sizes):
    """With rows of 2,048 and more, two correct bfloat16 computations do not stay one rounding step apart: some
    element of every vector lands on the other side of a rounding boundary at the first rounding, every
    product after it then moves all of its outputs a little, and after two layers the two differ by about as
    much as either differs from the exact result.  So the engine is held to the accuracy of the plain
    implementation that rounds to bfloat16 where the engine does: against the exact (double precision, unrounded)
    result its error may be at most 1.5 times (root mean square over the vocabulary) and 2 times (largest entry)
    the plain bfloat16 computation's own error at that position.  Positions whose routing the rounding can turn
    are left out: the gap between the last chosen and the first rejected expert moves by up to `turn` between
    the rounded and the exact computation, and positions with a gap below twice that are not compared."""
    cfg, eng, tensors, reqs = build("bfloat16", sizes)
    rounded = plain.PlainModel((cfg.to_dict(), tensors), compute=torch.float64, emulate_bf16=True, device="cuda")
    exact = plain.PlainModel((cfg.to_dict(), tensors), compute=torch.float64, device="cuda")
    del tensors
    ref_r = {rid: rounded.logits(t) for rid, t in reqs.items()}
    ref_e = {rid: exact.logits(t) for rid, t in reqs.items()}
    gap_r = {rid: rounded.router_margins(t) for rid, t in reqs.items()}
    gap_e = {rid: exact.router_margins(t) for rid, t in reqs.items()}
    turn = max(float((gap_r[rid] - gap_e[rid]).abs().max()) for rid in reqs)
    compared = total = 0
    for steps in cuttings_of(reqs):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(map(len, reqs.values()))
        for (rid, p), row in got.items():
            total += 1
            if min(float(gap_r[rid][p]), float(gap_e[rid][p])) < 2 * turn:
                continue
            own = ref_r[rid][p] - ref_e[rid][p]
            err = row - ref_e[rid][p]
            assert float(err.pow(2).mean().sqrt()) <= 1.5 * float(own.pow(2).mean().sqrt()), (rid, p)
            assert float(err.abs().max()) <= 2.0 * float(own.abs().max()), (rid, p)
            compared += 1
    print(f"compared {compared} of {total} positions (routing may turn within {turn:.2e})")
    assert compared >= FLOOR_BF16 * total, (compared, total, turn)
