"""The command line (options and lines after the reference's `dlm generate`, src/cli.rs:355-415,
src/main.rs:249-332): its parser and refusals on the CPU with the stand-in backend, and the
program itself as a child process on the GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen2_moe as plain
from plain_ops import PlainOps
from tiny_configs import TINY, prompt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _generated(out: str):
    return [json.loads(line.split(":", 1)[1]) for line in out.splitlines() if line.startswith("generated ids:")]


@pytest.fixture
def cpu_cli(monkeypatch):
    """cli.main with the engine on the stand-in backend (the program itself refuses the CPU)."""
    from dlm_b200 import cli
    from dlm_b200.engine import engine as engine_mod
    real = engine_mod.make_runtime
    monkeypatch.setattr(engine_mod, "make_runtime", lambda dtype, device, ops=None: real(dtype, "cpu", PlainOps()))
    return cli.main


def test_parser_defaults_are_the_references():
    from dlm_b200.cli import build_parser
    a = build_parser().parse_args(["generate"])
    assert (a.prompt, a.max_new_tokens, a.eos_token, a.seed, a.device) == (None, 16, None, 0, "gpu")   # cli.rs:355-415
    assert (a.vocab_size, a.hidden_size, a.num_layers, a.num_heads, a.num_kv_heads, a.intermediate_size) == \
        (32, 64, 2, 4, 2, 128)
    a = build_parser().parse_args(["generate", "--prompt", "1,2,3", "--prompt", "7"])
    assert a.prompt == [[1, 2, 3], [7]]
    with pytest.raises(SystemExit):
        build_parser().parse_args(["generate", "--prompt", "1,x"])


def test_refusals(cpu_cli, capsys, tiny_folders):
    assert cpu_cli(["generate", "--device", "cpu"]) == 2
    assert "no CPU path" in capsys.readouterr().err
    assert cpu_cli(["generate", "--prompt", ""]) == 2
    assert "empty" in capsys.readouterr().err
    assert cpu_cli(["generate", "--model-path", tiny_folders["A"], "--dtype", "fp32", "--prompt", "1,256"]) == 2
    assert "out of vocab range 256" in capsys.readouterr().err


def test_random_config_and_save_random(cpu_cli, capsys, tmp_path):
    """--random CONFIG.json builds whatever architecture the file names with seeded weights;
    --save-random writes that model as a folder; both generate what the oracle generates from
    the folder."""
    cfg_path = tmp_path / "b.json"
    cfg_path.write_text(json.dumps(TINY["B"]["cfg"]))
    p1, p2 = prompt(1, 9, 384), prompt(2, 20, 384)
    args = ["generate", "--dtype", "float32", "--page-size", "16", "--max-new-tokens", "6",
            "--prompt", ",".join(map(str, p1)), "--prompt", ",".join(map(str, p2))]
    assert cpu_cli(args + ["--random", str(cfg_path), "--seed", "1"]) == 0
    out = capsys.readouterr().out
    direct = _generated(out)
    assert f"prompt ids   : {p1}" in out and "3 layers" in out and "8 q-heads / 4 kv-heads" in out
    folder = tmp_path / "saved"
    assert cpu_cli(args + ["--random", str(cfg_path), "--seed", "1", "--save-random", str(folder)]) == 0
    saved = _generated(capsys.readouterr().out)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert cpu_cli(args + ["--model-path", str(folder)]) == 0
    loaded = _generated(capsys.readouterr().out)
    oracle = plain.PlainModel(str(folder), compute=torch.float64)
    want = [plain.generate(oracle, p, 6) for p in (p1, p2)]
    assert direct == saved == loaded == want
    # the demo geometry (the reference's options) goes through the registry as well
    assert cpu_cli(["generate", "--dtype", "float32", "--prompt", "1,2,3", "--max-new-tokens", "4", "--stats"]) == 0
    out = capsys.readouterr().out
    assert len(_generated(out)[0]) == 4 and "stats" in out and "not" in out


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_program_as_a_child_process(dtype, tiny_folders):
    """bin/dlm-b200 generate --model-path ... prints what Engine.generate returns."""
    from dlm_b200.engine import Engine
    V = TINY["D"]["cfg"]["vocab_size"]
    prompts = [prompt(5, 11, V), prompt(6, 40, V)]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "dlm-b200"), "generate", "--model-path", tiny_folders["D"],
           "--dtype", dtype, "--max-new-tokens", "12", "--stats"]
    for p in prompts:
        cmd += ["--prompt", ",".join(map(str, p))]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    eng = Engine.from_pretrained(tiny_folders["D"], dtype=dtype, page_size=64, num_pages=8, max_requests=2)
    assert _generated(run.stdout) == eng.generate(prompts, max_new_tokens=12)
    assert "device       : Gpu" in run.stdout
    bad = subprocess.run(cmd[:3] + ["--device", "cpu"], capture_output=True, text=True, timeout=600)
    assert bad.returncode == 2 and "no CPU path" in bad.stderr
