"""Weights by name: the reader, its errors, the one error that lists every fault, and the
random-weights mode."""
import json
import os
import struct

import pytest
import torch

from dlm_b200.parts.base import Runtime
from dlm_b200.parts.model import DecoderModel, WeightError
from dlm_b200.registry import resolve
from dlm_b200.weights import SafetensorsError, TensorStore, load_model, random_tensor, save_file, write_random_model
from tiny_configs import TINY, typed_config


def cpu_rt(dtype=torch.float32):
    return Runtime("cpu", dtype, ops=None)


def test_reader_agrees_with_safetensors_package(tiny_folders):
    from safetensors import safe_open
    store = TensorStore(tiny_folders["B"])
    with safe_open(os.path.join(tiny_folders["B"], "model.safetensors"), framework="pt") as sf:
        assert sorted(sf.keys()) == sorted(store.names())
        for k in list(sf.keys())[:25]:
            assert torch.equal(sf.get_tensor(k), store.tensor(k))
    store.close()


def test_round_trip_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.tensor(3.0)}
    path = str(tmp_path / "x.safetensors")
    save_file(t, path)
    st = TensorStore(path)
    for k, v in t.items():
        assert st.info(k) == (v.dtype, tuple(v.shape))
        assert torch.equal(st.tensor(k), v)


def test_malformed_files(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    with pytest.raises(SafetensorsError, match="no \\*.safetensors"):
        TensorStore(str(d))                               # src/storage/mmap_store.rs:168-173
    p = d / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        TensorStore(str(d))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        TensorStore(str(d))
    p.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(SafetensorsError, match="malformed header"):
        TensorStore(str(d))

    def write(header, data=b""):
        hj = json.dumps(header).encode()
        p.write_bytes(struct.pack("<Q", len(hj)) + hj + data)

    write({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside the file"):
        TensorStore(str(d))                               # src/storage/safetensors.rs:280-297
    write({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        TensorStore(str(d))
    write({"w": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 1]}}, b"\0")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        TensorStore(str(d))                               # src/storage/safetensors.rs:69-73


def test_one_error_lists_every_fault(tmp_path, tiny_folders):
    st = TensorStore(tiny_folders["A"])
    tensors = {n: st.tensor(n) for n in st.names()}
    del tensors["model.layers.1.mlp.experts.3.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(64, 65)
    tensors["model.layers.0.mlp.gate.weight"] = torch.zeros(7, 64)
    folder = tmp_path / "broken"
    folder.mkdir()
    save_file(tensors, str(folder / "model.safetensors"))
    with open(os.path.join(tiny_folders["A"], "config.json")) as f:
        (folder / "config.json").write_text(f.read())
    with pytest.raises(WeightError) as ei:
        load_model(str(folder), cpu_rt())
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.experts.3.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert sorted(n for n, _, _ in e.wrong_shape) == ["model.layers.0.mlp.gate.weight",
                                                      "model.layers.0.self_attn.o_proj.weight"]
    msg = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape: model.layers.0.mlp.gate.weight "
                   "is [7, 64], expected [8, 64]"):
        assert needle in msg


def test_load_keeps_dtypes_and_ties_head(tiny_folders):
    # matrices in the runtime dtype, norm weights and biases in 32-bit; no lm_head -> the embedding is the head
    cfg, model = load_model(tiny_folders["B"], cpu_rt(torch.bfloat16))
    assert model.lm_head is model.embed and model.embed.dtype == torch.bfloat16     # src/loader.rs:711-715
    attn = model.blocks[0].mixer
    assert attn.w_qkv.dtype == torch.bfloat16 and attn.w_qkv.shape == (256 + 2 * 128, 256)
    assert attn.b_qkv.dtype == torch.float32 and model.final_norm.weight.dtype == torch.float32
    cfg_a, model_a = load_model(tiny_folders["A"], cpu_rt())
    assert model_a.lm_head is not model_a.embed
    moe = model_a.blocks[0].ffn
    assert moe.w_gate_up.shape == (8, 64, 64) and moe.w_down.shape == (8, 64, 32) and moe.w_router.shape == (9, 64)
    st = TensorStore(tiny_folders["A"])
    g = st.tensor("model.layers.0.mlp.experts.5.gate_proj.weight")
    u = st.tensor("model.layers.0.mlp.experts.5.up_proj.weight")
    assert torch.equal(moe.w_gate_up[5, 0::2], g) and torch.equal(moe.w_gate_up[5, 1::2], u)


def test_bias_optional_by_presence(tmp_path, tiny_folders):
    st = TensorStore(tiny_folders["A"])
    tensors = {n: st.tensor(n) for n in st.names() if not n.endswith("_proj.bias")}
    folder = tmp_path / "nobias"
    folder.mkdir()
    save_file(tensors, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(open(os.path.join(tiny_folders["A"], "config.json")).read())
    _, model = load_model(str(folder), cpu_rt())
    assert model.blocks[0].mixer.b_qkv is None            # src/loader.rs:258-264


def test_shared_gate_optional_by_presence(tmp_path, tiny_folders):
    """A checkpoint without shared_expert_gate.weight loads; the shared expert then counts in full
    (src/forward/cpu.rs:1032-1041)."""
    st = TensorStore(tiny_folders["A"])
    tensors = {n: st.tensor(n) for n in st.names() if "shared_expert_gate" not in n}
    folder = tmp_path / "nogate"
    folder.mkdir()
    save_file(tensors, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(open(os.path.join(tiny_folders["A"], "config.json")).read())
    _, model = load_model(str(folder), cpu_rt())
    moe = model.blocks[0].ffn
    assert moe.has_gate is False and moe.w_router.shape == (8, 64) and moe.ws_down is not None
    _, with_gate = load_model(tiny_folders["A"], cpu_rt())
    assert with_gate.blocks[0].ffn.has_gate is True


def test_random_weights_are_a_function_of_seed_and_name(tmp_path):
    a = random_tensor("x.weight", (5, 7), "linear", 3)
    assert torch.equal(a, random_tensor("x.weight", (5, 7), "linear", 3))
    assert not torch.equal(a, random_tensor("x.weight", (5, 7), "linear", 4))
    assert not torch.equal(a, random_tensor("y.weight", (5, 7), "linear", 3))
    big = random_tensor("big", (400, 500), "linear", 0)
    assert abs(float(big.mean())) < 5e-4 and abs(float(big.std()) - 0.02) < 5e-4
    n = random_tensor("n", (20000,), "norm", 0)
    assert abs(float(n.mean()) - 1.0) < 1e-3 and abs(float(n.std()) - 0.02) < 1e-3
    # a prefix of a longer draw equals the shorter draw (values depend on the flat index only)
    assert torch.equal(random_tensor("p", (10,), "linear", 1), random_tensor("p", (100,), "linear", 1)[:10])


def test_written_folder_matches_spec(tmp_path):
    for name in TINY:
        folder = write_random_model(typed_config(name), TINY[name]["seed"], str(tmp_path / name))
        _, cfg, spec = resolve(folder)
        model = DecoderModel(spec, cpu_rt())
        st = TensorStore(folder)
        model.check({n: st.info(n) for n in st.names()})
        assert ("lm_head.weight" in st) == (not cfg.tie_word_embeddings)
