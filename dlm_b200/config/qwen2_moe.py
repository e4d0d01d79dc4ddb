"""Typed configuration of the Qwen2-MoE decoder (``Qwen2MoeForCausalLM``).

Every size and constant of the model comes from ``config.json`` through this
class; nothing downstream carries a literal size.  Keys, defaults and refusals
follow the reference's parser (src/model/config.rs:42-94, 235-274, 425-501);
the keys it does not read (``use_sliding_window``, ``sliding_window``,
``max_window_layers``, ``layer_types``, ``decoder_sparse_step``,
``mlp_only_layers``) and ``tie_word_embeddings`` are defined here.

Which layers are windowed: an explicit ``layer_types`` list (one of
``"full_attention"`` / ``"sliding_attention"`` per layer) wins when the key is
present; otherwise layer ``i`` is windowed iff ``use_sliding_window`` and
``i >= max_window_layers``.  (Other software that writes this key may derive
another default from ``max_window_layers``; a folder that carries the list is
therefore read by the list, never by the rule.)
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any

from .base import (ConfigError, as_bool, as_float, as_int, eos_list,
                   read_config_json, require_int)


LAYER_TYPES = ("full_attention", "sliding_attention")


def _layer_types(v: Any) -> list[str]:
    if not isinstance(v, (list, tuple)) or not all(isinstance(t, str) for t in v):
        raise ConfigError("layer_types must be a list of strings")
    return list(v)


@dataclass
class Qwen2MoeConfig:
    hidden_size: int
    num_attention_heads: int
    num_hidden_layers: int
    vocab_size: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    qkv_bias: bool | None = None   # None: decided by the presence of the bias tensors
    max_position_embeddings: int | None = None
    eos_token_ids: list[int] = field(default_factory=list)
    tie_word_embeddings: bool = False
    # mixture of experts (num_experts == 0: every layer is a dense MLP)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int | None = None
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: list[int] = field(default_factory=list)
    # sliding window
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int = 0
    layer_types: list[str] | None = None   # explicit per-layer choice; None: the max_window_layers rule

    architecture = "Qwen2MoeForCausalLM"
    model_type = "qwen2_moe"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen2MoeConfig":
        if raw.get("quantization_config") is not None:
            raise ConfigError("quantization_config is present: quantized checkpoints are not supported")
        rs = raw.get("rope_scaling")
        if rs is not None:
            kind = ""
            if isinstance(rs, dict):
                kind = str(rs.get("rope_type", rs.get("type", "")) or "").lower()
            if kind not in ("", "default"):
                raise ConfigError(
                    f"rope_scaling type {kind!r} is not implemented; running the model without "
                    "its trained scaling would give incoherent output, so it is refused")
        hidden = require_int(raw, "hidden_size")
        nh = require_int(raw, "num_attention_heads")
        layers = require_int(raw, "num_hidden_layers")
        vocab = require_int(raw, "vocab_size")
        nkv = as_int(raw["num_key_value_heads"], "num_key_value_heads", minimum=1) \
            if raw.get("num_key_value_heads") is not None else nh
        if raw.get("head_dim") is not None:
            hd = as_int(raw["head_dim"], "head_dim", minimum=1)
        else:
            if hidden % nh != 0:
                raise ConfigError(f"hidden_size ({hidden}) is not divisible by num_attention_heads ({nh})")
            hd = hidden // nh
        inter = as_int(raw["intermediate_size"], "intermediate_size", minimum=1) \
            if raw.get("intermediate_size") is not None else 4 * hidden
        n_exp = as_int(raw["num_experts"], "num_experts", minimum=0) if raw.get("num_experts") is not None else 0
        topk = 0
        moe_inter = 0
        shared = None
        if n_exp > 0:
            if raw.get("num_experts_per_tok") is None:
                raise ConfigError("config declares experts but no num_experts_per_tok; "
                                  "the routing top-k is never guessed")
            topk = as_int(raw["num_experts_per_tok"], "num_experts_per_tok", minimum=1)
            moe_inter = as_int(raw["moe_intermediate_size"], "moe_intermediate_size", minimum=1) \
                if raw.get("moe_intermediate_size") is not None else inter
            if raw.get("shared_expert_intermediate_size") is not None:
                shared = as_int(raw["shared_expert_intermediate_size"], "shared_expert_intermediate_size", minimum=0)
                if shared == 0:
                    shared = None
        cfg = cls(
            hidden_size=hidden, num_attention_heads=nh, num_hidden_layers=layers, vocab_size=vocab,
            num_key_value_heads=nkv, head_dim=hd, intermediate_size=inter,
            rope_theta=as_float(raw["rope_theta"], "rope_theta") if raw.get("rope_theta") is not None else 10000.0,
            rms_norm_eps=as_float(raw["rms_norm_eps"], "rms_norm_eps") if raw.get("rms_norm_eps") is not None else 1e-5,
            qkv_bias=as_bool(raw["qkv_bias"], "qkv_bias") if raw.get("qkv_bias") is not None else None,
            max_position_embeddings=as_int(raw["max_position_embeddings"], "max_position_embeddings", minimum=1)
            if raw.get("max_position_embeddings") is not None else None,
            eos_token_ids=eos_list(raw.get("eos_token_id")),
            tie_word_embeddings=as_bool(raw["tie_word_embeddings"], "tie_word_embeddings")
            if raw.get("tie_word_embeddings") is not None else False,
            num_experts=n_exp, num_experts_per_tok=topk, moe_intermediate_size=moe_inter,
            shared_expert_intermediate_size=shared,
            norm_topk_prob=as_bool(raw["norm_topk_prob"], "norm_topk_prob")
            if raw.get("norm_topk_prob") is not None else True,
            decoder_sparse_step=as_int(raw["decoder_sparse_step"], "decoder_sparse_step", minimum=1)
            if raw.get("decoder_sparse_step") is not None else 1,
            mlp_only_layers=[as_int(i, "mlp_only_layers[]") for i in (raw.get("mlp_only_layers") or [])],
            use_sliding_window=as_bool(raw["use_sliding_window"], "use_sliding_window")
            if raw.get("use_sliding_window") is not None else False,
            sliding_window=as_int(raw["sliding_window"], "sliding_window", minimum=1)
            if raw.get("sliding_window") is not None else None,
            max_window_layers=as_int(raw["max_window_layers"], "max_window_layers", minimum=0)
            if raw.get("max_window_layers") is not None else 0,
            layer_types=_layer_types(raw["layer_types"]) if raw.get("layer_types") is not None else None,
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen2MoeConfig":
        return cls.from_dict(read_config_json(path))

    # --------------------------------------------------------------- validate
    def validate(self) -> None:
        for key in ("hidden_size", "num_attention_heads", "num_hidden_layers", "vocab_size",
                    "num_key_value_heads", "head_dim", "intermediate_size"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be > 0")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even (rotary pairs)")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                              f"num_key_value_heads ({self.num_key_value_heads})")
        if not (self.rms_norm_eps >= 0.0):
            raise ConfigError("rms_norm_eps must be >= 0")
        if not (self.rope_theta > 0.0):
            raise ConfigError("rope_theta must be > 0")
        if self.num_experts > 0:
            if not (1 <= self.num_experts_per_tok <= self.num_experts):
                raise ConfigError(f"num_experts_per_tok ({self.num_experts_per_tok}) must be in "
                                  f"1..={self.num_experts}")
            if self.moe_intermediate_size <= 0:
                raise ConfigError("moe_intermediate_size must be > 0")
        for i in self.mlp_only_layers:
            if not (0 <= i < self.num_hidden_layers):
                raise ConfigError(f"mlp_only_layers entry {i} is outside 0..{self.num_hidden_layers - 1}")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("use_sliding_window is true but sliding_window is missing or not > 0")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(f"layer_types has {len(self.layer_types)} entries, the model has "
                                  f"{self.num_hidden_layers} layers")
            for i, t in enumerate(self.layer_types):
                if t not in LAYER_TYPES:
                    raise ConfigError(f"layer_types[{i}] is {t!r}; known: {list(LAYER_TYPES)}")
            if "sliding_attention" in self.layer_types and (self.sliding_window is None or self.sliding_window <= 0):
                raise ConfigError("layer_types names a sliding_attention layer but sliding_window is missing or not > 0")
        for t in self.eos_token_ids:
            if t < 0:
                raise ConfigError("eos_token_id must be >= 0")

    # ------------------------------------------------------------- per layer
    def layer_is_sparse(self, i: int) -> bool:
        """Layer ``i`` routes through experts iff the model has experts, ``i`` is not in
        ``mlp_only_layers`` and ``(i + 1) % decoder_sparse_step == 0``; otherwise it is a
        dense SwiGLU MLP of width ``intermediate_size``."""
        return (self.num_experts > 0 and i not in self.mlp_only_layers
                and (i + 1) % self.decoder_sparse_step == 0)

    def layer_window(self, i: int) -> int | None:
        """The window of layer ``i`` (it sees only the last ``sliding_window`` positions, itself
        included) or None.  ``layer_types[i]`` decides when the list is given; otherwise the layer
        is windowed iff ``use_sliding_window`` and ``i >= max_window_layers``."""
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[i] == "sliding_attention" else None
        if self.use_sliding_window and i >= self.max_window_layers:
            return self.sliding_window
        return None

    # ------------------------------------------------------------------ dump
    def to_dict(self) -> dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        eos = d.pop("eos_token_ids")
        if len(eos) == 1:
            d["eos_token_id"] = eos[0]
        elif eos:
            d["eos_token_id"] = list(eos)
        if d["num_experts"] == 0:
            for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size",
                      "shared_expert_intermediate_size", "norm_topk_prob"):
                d.pop(k)
        d = {k: v for k, v in d.items() if v is not None}
        d["architectures"] = [self.architecture]
        d["model_type"] = self.model_type
        return d
