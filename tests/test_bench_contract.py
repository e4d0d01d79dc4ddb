"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line and exit
code 2, the reference arm prints its `unavailable` line and exits 0, and the helper arithmetic of the
roofline holds for a hand-made case."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          env={**os.environ, **(env or {})}, timeout=120)


def test_more_than_one_gpu_is_refused():
    r = run("--gpus", "2")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]
    r = run(env={"WORLD_SIZE": "4"})
    assert r.returncode == 2


def test_reference_arm_says_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_roofline_bytes_of_a_hand_made_case():
    sys.path.insert(0, ROOT)
    import bench
    from dlm_b200.config import Qwen2MoeConfig
    raw = dict(bench.MODEL)
    raw.update(num_hidden_layers=1, hidden_size=8, num_attention_heads=2, num_key_value_heads=1, head_dim=4,
               num_experts=4, num_experts_per_tok=2, moe_intermediate_size=6, shared_expert_intermediate_size=10,
               vocab_size=32)
    cfg = Qwen2MoeConfig.from_dict(raw)
    got = bench.weight_bytes_per_decode_step(cfg, batch=1, layers=1, esz=2)
    H, qkv, o = 8, (2 + 2 * 1) * 4 * 8, 8 * 8
    routed = 2 * 3 * 8 * 6              # two experts with rows, gate + up + down
    shared = 3 * 8 * 10
    head = 32 * 8
    # at least every matrix that one token uses, once; nothing the size of the whole expert table
    assert got >= 2 * (qkv + o + routed + shared + head)
    assert got < 2 * (qkv + o + 4 * 3 * 8 * 6 + shared + head) + 4096
