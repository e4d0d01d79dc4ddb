"""bin/trace_run as a user runs it: a child process fed steps on standard input, one at a
time, each after the previous ``done``; its files are compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import cuttings
import plain_qwen2_moe as plain
from tiny_configs import TINY, prompt

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 1e-4, "bfloat16": 1e-2}
# positions whose routing is a near-tie for the precision under test are not compared (see test_engine_gpu.py)
MARGIN = {"float32": 1e-6, "bfloat16": 2e-4}


def replay(folder, dtype, steps, out_dir, max_tokens, env=None):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1,
                            env=None if env is None else {**os.environ, **env})
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


def read_logits(out_dir, steps, vocab):
    got, fed = {}, {}
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            for e in st["entries"]:
                fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
            continue
        arr = np.fromfile(path, dtype="<f4")
        assert arr.size == wanted * vocab
        arr = torch.from_numpy(arr.reshape(wanted, vocab).copy())
        row = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = arr[row]
                row += 1
            fed[e["id"]] = base + len(e["tokens"])
    return got


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_mixed(name, dtype, tiny_folders, tmp_path):
    V = TINY[name]["cfg"]["vocab_size"]
    oracle = plain.PlainModel(tiny_folders[name], compute=torch.float64, emulate_bf16=(dtype == "bfloat16"))
    toks = {f"q{i}": prompt(200 + i, n, V) for i, n in enumerate([70, 33, 100, 16, 90, 5])}
    margins = {rid: oracle.router_margins(t) for rid, t in toks.items()}
    steps, _ = cuttings.mixed(toks, max_live=4, seed=9)
    # some entries ask for nothing, some for a part
    for i, st in enumerate(steps):
        if i % 5 == 1:
            for e in st["entries"]:
                if len(e["tokens"]) > 1:
                    e["want"] = e["want"][-1:]
    peak = cuttings.peak_tokens(steps)
    out_dir = str(tmp_path / "out")
    replay(tiny_folders[name], dtype, steps, out_dir, peak)
    got = read_logits(out_dir, steps, V)
    assert got, "no logits were written"
    checked = 0
    full = {rid: oracle.logits(t) for rid, t in toks.items()}
    for (rid, p), row in got.items():
        if float(margins[rid][p]) < MARGIN[dtype]:
            continue
        ref = full[rid][p]
        d = float((row - ref).abs().max())
        assert d <= TOL[dtype], f"{rid} position {p}: {d:.3e}"
        checked += 1
    assert checked > 0.5 * len(got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_launches_change_no_bit(dtype, tiny_folders, tmp_path):
    """Kernels that start while the kernel before them ends, and the shared expert on a second stream, only
    move work in time: with both switched off the same trace gives the same bits."""
    name = "B"
    V = TINY[name]["cfg"]["vocab_size"]
    toks = {f"q{i}": prompt(300 + i, n, V) for i, n in enumerate([70, 33, 100, 16])}
    steps, _ = cuttings.mixed(toks, max_live=4, seed=11)
    peak = cuttings.peak_tokens(steps)
    outs = []
    for tag, env in (("on", None), ("off", {"DLM_B200_NO_PDL": "1", "DLM_B200_NO_BRANCH": "1"})):
        out_dir = str(tmp_path / tag)
        replay(tiny_folders[name], dtype, steps, out_dir, peak, env=env)
        outs.append(read_logits(out_dir, steps, V))
    assert outs[0].keys() == outs[1].keys() and outs[0]
    for key in outs[0]:
        assert torch.equal(outs[0][key], outs[1][key]), f"{key} differs"


@pytest.mark.parametrize("switch", ["DLM_B200_NO_PAIR", "DLM_B200_NO_TCGEN05", "DLM_B200_NO_STREAM"])
def test_older_kernels_give_the_same_answers(switch, tiny_folders, tmp_path):
    """Each switch that takes an older kernel (single-SM tcgen05 products, warp-level MMA and cp.async instead
    of tcgen05 and TMA, per-lane loads instead of bulk copies) leaves the logits within the bfloat16 tolerance
    of the plain implementation: a fault in a fallback does not wait for the day it is needed."""
    name, dtype = "D", "bfloat16"       # head_dim 128: the tcgen05 attention and the TMA decode attention are in play
    V = TINY[name]["cfg"]["vocab_size"]
    oracle = plain.PlainModel(tiny_folders[name], compute=torch.float64, emulate_bf16=True)
    toks = {f"q{i}": prompt(400 + i, n, V) for i, n in enumerate([150, 40, 97, 20])}
    margins = {rid: oracle.router_margins(t) for rid, t in toks.items()}
    steps, _ = cuttings.mixed(toks, max_live=4, seed=13)
    peak = cuttings.peak_tokens(steps)
    out_dir = str(tmp_path / "out")
    replay(tiny_folders[name], dtype, steps, out_dir, peak, env={switch: "1"})
    got = read_logits(out_dir, steps, V)
    assert got, "no logits were written"
    full = {rid: oracle.logits(t) for rid, t in toks.items()}
    checked = 0
    for (rid, p), row in got.items():
        if float(margins[rid][p]) < MARGIN[dtype]:
            continue
        d = float((row - full[rid][p]).abs().max())
        assert d <= TOL[dtype], f"{switch}: {rid} position {p}: {d:.3e}"
        checked += 1
    assert checked > 0.5 * len(got)
