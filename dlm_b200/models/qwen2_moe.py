"""Qwen2-MoE (``Qwen2MoeForCausalLM``) as a ``ModelSpec`` of parts.

Per layer, from the config: attention with or without a sliding window
(``layer_window``), and a routed mixture of experts or a dense MLP
(``layer_is_sparse``).  A shared expert whose gate tensor the checkpoint lacks
is taken with the factor 1, as the reference does (src/forward/cpu.rs:1032-1041).  Tensor names are the checkpoint's own
(src/loader.rs:392-418, 434-453): nothing is renamed.
"""
from __future__ import annotations

from ..config.qwen2_moe import Qwen2MoeConfig
from ..parts.base import PartSpec
from ..parts.model import ModelSpec
from ..registry import register_architecture

_NAMES = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.", "ffn": "mlp."}


def build_spec(cfg: Qwen2MoeConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    rope = PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    layers, prefixes = [], []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "qkv_bias": cfg.qkv_bias, "window": cfg.layer_window(i), "position": rope})
        if cfg.layer_is_sparse(i):
            ffn = PartSpec("moe_softmax_topk", {
                "hidden_size": cfg.hidden_size, "num_experts": cfg.num_experts, "top_k": cfg.num_experts_per_tok,
                "expert_intermediate_size": cfg.moe_intermediate_size, "norm_topk_prob": cfg.norm_topk_prob,
                "shared_intermediate_size": cfg.shared_expert_intermediate_size, "shared_gate": None})
        else:
            ffn = PartSpec("swiglu_dense", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        layers.append(PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn, "names": _NAMES}))
        prefixes.append(f"model.layers.{i}.")
    return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, layers=layers, layer_prefixes=prefixes,
                     final_norm=norm, tie_word_embeddings=cfg.tie_word_embeddings)


register_architecture(Qwen2MoeConfig.architecture, Qwen2MoeConfig, build_spec, model_type=Qwen2MoeConfig.model_type)
