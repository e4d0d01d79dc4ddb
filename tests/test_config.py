"""Configuration and registry (cases after the reference's tests/phase1.rs:168-226)."""
import json

import pytest

from dlm_b200 import registry
from dlm_b200.config import ConfigError, Qwen2MoeConfig
from tiny_configs import TINY

BASE = dict(architectures=["Qwen2MoeForCausalLM"], hidden_size=64, num_attention_heads=4, num_hidden_layers=2,
            vocab_size=100)


def test_defaults_follow_the_reference():
    c = Qwen2MoeConfig.from_dict(BASE)
    assert c.num_key_value_heads == 4          # src/model/config.rs:444
    assert c.intermediate_size == 256          # 4 * hidden, config.rs:447-449
    assert c.head_dim == 16                    # config.rs:505-508
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5    # config.rs:456-457
    assert c.num_experts == 0 and not c.layer_is_sparse(0)
    assert c.eos_token_ids == [] and c.qkv_bias is None


def test_eos_scalar_list_and_generation_config(tmp_path):
    assert Qwen2MoeConfig.from_dict({**BASE, "eos_token_id": 7}).eos_token_ids == [7]
    assert Qwen2MoeConfig.from_dict({**BASE, "eos_token_id": [7, 9]}).eos_token_ids == [7, 9]
    (tmp_path / "config.json").write_text(json.dumps({**BASE, "eos_token_id": 7}))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 11]}))
    assert Qwen2MoeConfig.from_json(str(tmp_path)).eos_token_ids == [7, 11]


def test_moe_keys():
    moe = {**BASE, "num_experts": 8, "num_experts_per_tok": 2, "intermediate_size": 96}
    c = Qwen2MoeConfig.from_dict(moe)
    assert c.moe_intermediate_size == 96 and c.norm_topk_prob is True     # config.rs:257-264, 271
    assert Qwen2MoeConfig.from_dict({**moe, "norm_topk_prob": False}).norm_topk_prob is False
    with pytest.raises(ConfigError, match="num_experts_per_tok"):
        Qwen2MoeConfig.from_dict({**BASE, "num_experts": 8})               # config.rs:244-250
    with pytest.raises(ConfigError):
        Qwen2MoeConfig.from_dict({**moe, "num_experts_per_tok": 9})
    assert Qwen2MoeConfig.from_dict({**BASE, "num_experts": 0}).num_experts == 0


def test_layer_rules():
    b = Qwen2MoeConfig.from_dict(TINY["B"]["cfg"])
    assert [b.layer_is_sparse(i) for i in range(3)] == [False, True, False]
    assert [b.layer_window(i) for i in range(3)] == [None, 16, 16]
    a = Qwen2MoeConfig.from_dict(TINY["A"]["cfg"])
    assert all(a.layer_is_sparse(i) for i in range(2)) and a.layer_window(1) is None


def test_layer_types_win_over_the_rule():
    raw = {**TINY["B"]["cfg"], "layer_types": ["sliding_attention", "full_attention", "sliding_attention"]}
    c = Qwen2MoeConfig.from_dict(raw)
    assert [c.layer_window(i) for i in range(3)] == [16, None, 16]
    # the list decides even when use_sliding_window is false
    c = Qwen2MoeConfig.from_dict({**raw, "use_sliding_window": False})
    assert [c.layer_window(i) for i in range(3)] == [16, None, 16]
    spec = registry.resolve(raw)[2]
    assert [s.params["mixer"].params["window"] for s in spec.layers] == [16, None, 16]
    assert Qwen2MoeConfig.from_dict(c.to_dict()) == c
    # without the key: layer i is windowed iff use_sliding_window and i >= max_window_layers
    c = Qwen2MoeConfig.from_dict(TINY["B"]["cfg"])
    assert c.layer_types is None and [c.layer_window(i) for i in range(3)] == [None, 16, 16]
    with pytest.raises(ConfigError, match="layer_types has 2"):
        Qwen2MoeConfig.from_dict({**raw, "layer_types": ["full_attention"] * 2})
    with pytest.raises(ConfigError, match="chunked"):
        Qwen2MoeConfig.from_dict({**raw, "layer_types": ["chunked", "full_attention", "full_attention"]})
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2MoeConfig.from_dict({**BASE, "layer_types": ["sliding_attention", "full_attention"]})
    with pytest.raises(ConfigError, match="list of strings"):
        Qwen2MoeConfig.from_dict({**raw, "layer_types": "sliding_attention"})


@pytest.mark.parametrize("patch,match", [
    ({"num_attention_heads": 0}, "num_attention_heads"),
    ({"hidden_size": 66}, "divisible"),
    ({"head_dim": 15}, "even"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"quantization_config": {"bits": 4}}, "quantiz"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"mlp_only_layers": [5]}, "mlp_only_layers"),
    ({"vocab_size": "big"}, "vocab_size"),
])
def test_refusals(patch, match):
    with pytest.raises(ConfigError, match=match):
        Qwen2MoeConfig.from_dict({**BASE, **patch})


def test_missing_key_and_bad_json(tmp_path):
    bad = dict(BASE)
    del bad["hidden_size"]
    with pytest.raises(ConfigError, match="hidden_size"):
        Qwen2MoeConfig.from_dict(bad)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        Qwen2MoeConfig.from_json(str(tmp_path))
    with pytest.raises(ConfigError, match="no config.json"):
        Qwen2MoeConfig.from_json(str(tmp_path / "nowhere"))


def test_registry():
    assert "Qwen2MoeForCausalLM" in registry.architectures()
    name, cfg, spec = registry.resolve(dict(TINY["B"]["cfg"]))
    assert name == "Qwen2MoeForCausalLM" and isinstance(cfg, Qwen2MoeConfig)
    assert [s.params["ffn"].kind for s in spec.layers] == ["swiglu_dense", "moe_softmax_topk", "swiglu_dense"]
    assert [s.params["mixer"].params["window"] for s in spec.layers] == [None, 16, 16]
    by_type = dict(TINY["A"]["cfg"])
    del by_type["architectures"]
    assert registry.resolve(by_type)[0] == "Qwen2MoeForCausalLM"
    with pytest.raises(ConfigError, match="registered"):
        registry.resolve({**BASE, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="names no architecture"):
        registry.resolve({k: v for k, v in BASE.items() if k != "architectures"})


def test_round_trip():
    for name in TINY:
        c = Qwen2MoeConfig.from_dict(TINY[name]["cfg"])
        assert Qwen2MoeConfig.from_dict(c.to_dict()) == c
