"""Tiny Qwen2-MoE configurations for the tests.  A and B differ in every size and option
(heads and groups, head size, widths that are no power of two, layers, vocabulary, eps,
rope base, window, experts and top-k, renormalisation, dense layers, tied head); C adds
an explicit head_dim that is not hidden/heads, a single kv head and no shared expert; D has
the head size (128) and widths (multiples of 8) that the tcgen05 attention and GEMM kernels take,
so that the engine tests reach them with pages of 64 tokens and prompts above 128 tokens."""
import torch

TINY = {
    "A": dict(seed=0, cfg=dict(
        architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
        num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
        num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=64,
        norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=128,
        vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, use_sliding_window=False,
        tie_word_embeddings=False)),
    "B": dict(seed=1, cfg=dict(
        architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
        num_hidden_layers=3, hidden_size=256, num_attention_heads=8, num_key_value_heads=4,
        num_experts=12, num_experts_per_tok=3, moe_intermediate_size=48, shared_expert_intermediate_size=96,
        norm_topk_prob=True, decoder_sparse_step=2, mlp_only_layers=[0], intermediate_size=160,
        vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5, use_sliding_window=True, sliding_window=16,
        max_window_layers=1, tie_word_embeddings=True)),
    "C": dict(seed=2, cfg=dict(
        architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
        num_hidden_layers=2, hidden_size=72, num_attention_heads=3, num_key_value_heads=1, head_dim=48,
        num_experts=5, num_experts_per_tok=1, moe_intermediate_size=40,
        norm_topk_prob=True, decoder_sparse_step=1, intermediate_size=88,
        vocab_size=301, rope_theta=50000.0, rms_norm_eps=3e-6, use_sliding_window=True, sliding_window=24,
        max_window_layers=0, tie_word_embeddings=False)),
    "D": dict(seed=3, cfg=dict(
        architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
        num_hidden_layers=2, hidden_size=192, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
        num_experts=6, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=128,
        norm_topk_prob=False, decoder_sparse_step=1, intermediate_size=96,
        vocab_size=520, rope_theta=20000.0, rms_norm_eps=2e-6, use_sliding_window=True, sliding_window=40,
        max_window_layers=1, tie_word_embeddings=False)),
}


def typed_config(name):
    from dlm_b200.config import Qwen2MoeConfig
    return Qwen2MoeConfig.from_dict(TINY[name]["cfg"])


def write_tiny(name, out_dir, dtype=torch.float32):
    from dlm_b200.weights import write_random_model
    return write_random_model(typed_config(name), TINY[name]["seed"], out_dir, dtype=dtype)


def prompt(seed, length, vocab):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()

