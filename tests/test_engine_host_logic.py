"""The engine's host side without a GPU: the cache, the step function's bookkeeping, the
scheduler loop and the replay program, with the plain PyTorch statement of the kernels
(tests/plain_ops.py) standing in for them.  This checks the logic, not the kernels; the
product has no such backend."""
import io
import json
import os
import sys

import numpy as np
import pytest
import torch

import cuttings
import plain_qwen2_moe as plain
from plain_ops import PlainOps
from tiny_configs import TINY, prompt


@pytest.fixture(scope="module")
def oracles(tiny_folders):
    return {n: plain.PlainModel(tiny_folders[n], compute=torch.float64) for n in TINY}


def engine(folder, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=40, max_requests=8)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


@pytest.mark.parametrize("name", list(TINY))
def test_every_cutting_matches_the_oracle(name, tiny_folders, oracles):
    V = TINY[name]["cfg"]["vocab_size"]
    reqs = {f"r{i}": prompt(i, n, V) for i, n in enumerate([1, 16, 33, 70])}
    ref = {rid: oracles[name].logits(t) for rid, t in reqs.items()}
    eng = engine(tiny_folders[name])
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=1)
    for steps in (cuttings.whole(reqs), cuttings.tail_decode(reqs, 20), cuttings.portions(reqs), mixed):
        got = cuttings.run_trace(eng, steps)
        for (rid, p), row in got.items():
            assert float((row - ref[rid][p]).abs().max()) < 1e-4
        assert len(got) == sum(len(t) for t in reqs.values())


def test_pages_are_reused_and_window_pages_return(tiny_folders, oracles):
    V = TINY["B"]["cfg"]["vocab_size"]
    reqs = {f"r{i}": prompt(10 + i, n, V) for i, n in enumerate([70, 33, 129, 16, 90, 7])}
    steps, _ = cuttings.mixed(reqs, max_live=3, seed=2)
    peak = cuttings.peak_tokens(steps)
    eng = engine(tiny_folders["B"], num_pages=peak // 16)
    got = cuttings.run_trace(eng, steps)
    for (rid, p), row in got.items():
        assert float((row - oracles["B"].logits(reqs[rid][:p + 1])[-1]).abs().max()) < 1e-4
    full, windowed = eng.cache.stats()
    assert full.used_pages == 0 and windowed.used_pages == 0
    assert windowed.high_water < full.high_water          # the window group needed fewer pages


def test_generate_equals_oracle_and_batched_equals_isolated(tiny_folders, oracles):
    V = TINY["A"]["cfg"]["vocab_size"]
    prompts = [prompt(20 + i, n, V) for i, n in enumerate([1, 7, 16, 33])]
    eng = engine(tiny_folders["A"], max_requests=2, max_step_tokens=12)
    outs = eng.generate(prompts, max_new_tokens=10)
    for p, o in zip(prompts, outs):
        assert o == plain.generate(oracles["A"], p, 10)
    assert eng.generate(prompts[2], max_new_tokens=10) == outs[2]
    stop = outs[1][4]
    assert eng.generate(prompts[1], max_new_tokens=10, eos_token=stop) == outs[1][:outs[1].index(stop) + 1]
    sampled = eng.generate(prompts, max_new_tokens=10, temperature=0.8, seed=3)
    assert sampled == [eng.generate(p, max_new_tokens=10, temperature=0.8, seed=3) for p in prompts]
    assert eng.stats()["pages"][0]["used"] == 0
    with pytest.raises(ValueError):
        eng.generate([[]])
    with pytest.raises(ValueError):
        eng.generate([[V]])


def test_named_twice_and_shared_cache(tiny_folders, oracles):
    """The order of layers is data: [0, 1, 0] runs layer 0 twice (each call with a cache of
    its own); a call may also read the cache an earlier call wrote."""
    from dlm_b200.engine import Engine
    from dlm_b200.parts.base import Runtime
    from dlm_b200.parts.model import DecoderModel, LayerCall
    from dlm_b200.registry import resolve
    from dlm_b200.weights import TensorStore
    folder = tiny_folders["A"]
    _, cfg, spec = resolve(folder)
    spec.order = [LayerCall(0), LayerCall(1), LayerCall(0)]
    model = DecoderModel(spec, Runtime("cpu", torch.float32, PlainOps()))
    st = TensorStore(folder)
    model.load(st.tensor, st.names())
    eng = Engine(cfg, model, page_size=16, num_pages=16, max_requests=2)
    toks = prompt(5, 40, cfg.vocab_size)
    ref = oracles["A"].logits(toks, layer_order=[0, 1, 0])
    s = eng.cache.open()
    a = eng.step([(s, toks[:23], list(range(23)))])
    b = eng.step([(s, toks[23:], list(range(17)))])
    assert float((torch.cat([a, b]) - ref).abs().max()) < 1e-4
    assert len(eng.cache.k) == 3
    # call 2 reads call 0's keys and values instead of writing its own: two caches, and the result differs
    spec.order = [LayerCall(0), LayerCall(1), LayerCall(0, reads_cache_of=0)]
    model2 = DecoderModel(spec, Runtime("cpu", torch.float32, PlainOps()))
    model2.load(st.tensor, st.names())
    eng2 = Engine(cfg, model2, page_size=16, num_pages=16, max_requests=2)
    s2 = eng2.cache.open()
    c = eng2.step([(s2, toks, list(range(40)))])
    assert len(eng2.cache.k) == 2 and c.shape == ref.shape and float((c - ref).abs().max()) > 1e-4
    s3 = eng2.cache.open()
    d = torch.cat([eng2.step([(s3, toks[:9], list(range(9)))]), eng2.step([(s3, toks[9:], list(range(31)))])])
    assert float((c - d).abs().max()) < 1e-5
    with pytest.raises(ValueError):
        spec.order = [LayerCall(0, reads_cache_of=1), LayerCall(1)]
        DecoderModel(spec, Runtime("cpu", torch.float32, PlainOps()))


def test_replay_program_protocol(tiny_folders, oracles, tmp_path, monkeypatch, capsys):
    """The replay program's own loop (here in-process, on the stand-in backend)."""
    from dlm_b200.engine import engine as engine_mod
    from dlm_b200.engine import replay
    V = TINY["A"]["cfg"]["vocab_size"]
    a, b = prompt(1, 20, V), prompt(2, 9, V)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:12], "want": [0, 11]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[12:14], "want": []}, {"id": "b", "tokens": b, "want": [8]}],
         "end": ["b"]},
        {"step": 2, "entries": [], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[14:], "want": [5]}], "end": ["a"]},
    ]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    real = engine_mod.make_runtime
    monkeypatch.setattr(engine_mod, "make_runtime", lambda dtype, device, ops=None: real(dtype, "cpu", PlainOps()))
    out = tmp_path / "out"
    rc = replay.main(["--model", tiny_folders["A"], "--dtype", "float32", "--out", str(out), "--max-tokens", "128",
                      "--device", "cpu"])
    assert rc == 0
    assert capsys.readouterr().out.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "3.f32"]
    ra, rb = oracles["A"].logits(a), oracles["A"].logits(b)
    l0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V))
    l1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    l3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4").reshape(1, V))
    assert float((l0 - ra[[0, 11]]).abs().max()) < 1e-4
    assert float((l1 - rb[[8]]).abs().max()) < 1e-4
    assert float((l3 - ra[[19]]).abs().max()) < 1e-4


def test_gateless_shared_expert_and_explicit_layer_types(tiny_folders, tmp_path):
    """A checkpoint without the shared expert's gate tensor runs with the factor 1
    (src/forward/cpu.rs:1032-1041), and an explicit layer_types list decides which layers are
    windowed; both against the oracle, which reads the same folder on its own."""
    import shutil
    from safetensors.torch import load_file, save_file
    V = TINY["B"]["cfg"]["vocab_size"]
    folder = tmp_path / "variant"
    shutil.copytree(tiny_folders["B"], folder)
    tensors = {n: t for n, t in load_file(str(folder / "model.safetensors")).items() if "shared_expert_gate" not in n}
    save_file(tensors, str(folder / "model.safetensors"))
    raw = json.loads((folder / "config.json").read_text())
    raw["layer_types"] = ["sliding_attention", "full_attention", "sliding_attention"]
    (folder / "config.json").write_text(json.dumps(raw))
    oracle = plain.PlainModel(str(folder), compute=torch.float64)
    toks = prompt(3, 60, V)
    ref = oracle.logits(toks)
    base = plain.PlainModel(tiny_folders["B"], compute=torch.float64).logits(toks)
    assert float((ref - base).abs().max()) > 1e-3          # the variant is another model
    eng = engine(str(folder))
    assert [b.mixer.window for b in eng.model.blocks] == [16, None, 16]
    assert eng.model.blocks[1].ffn.has_gate is False
    got = cuttings.run_trace(eng, cuttings.portions({"r": toks}))
    for (rid, p), row in got.items():
        assert float((row - ref[p]).abs().max()) < 1e-4
