"""Makes the golden hidden states under tests/golden/ by running the reference's own CUDA
model code (vedantnimbarte/dlm, src/gpu/kernels.cu: dlm_decode_block, dlm_moe_attn,
dlm_moe_matvec, dlm_apply_expert) on tiny random Qwen2-MoE models, one token at a time, the
way the reference's host drives them (src/forward/streaming_gpu.rs:577-712 for a layer of
experts, src/forward/gpu.rs for a dense layer).

The reference is a Rust crate and no Rust toolchain exists where these tests run, but its
kernel file is plain CUDA C++ with extern "C" entry points: nvcc compiles it unchanged and
this script calls it through ctypes.  What the Rust host does between the calls is restated
here (route_topk, src/forward/cpu.rs:980-999, in 32-bit floats; the shared expert's sigmoid,
streaming_gpu.rs:672-690): a softmax over all router logits, the k largest, renormalised or not.

The reference has no sliding window, so the tiny configurations are run with the window
switched off; it has neither decoder_sparse_step nor mlp_only_layers, so which entry point a
layer gets follows the rule under test ((i + 1) % step == 0 and i not in mlp_only_layers).
The golden files therefore pin: embedding, RMS norm, q/k/v with bias, rotary pairs and
angles, grouped-query attention, the SwiGLU expert, routing weights and order, the shared
expert and its gate.  tests/test_golden.py compares tests/plain_qwen2_moe.py with them.

Usage (needs a CUDA device and nvcc; run once, outputs are committed):

    python tests/golden/make_golden.py --kernels-cu <reference>/src/gpu/kernels.cu --out tests/golden
"""
import argparse
import ctypes
import hashlib
import json
import math
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

PROMPT_LEN = 24


def compile_reference(cu_path: str, workdir: str) -> ctypes.CDLL:
    so = os.path.join(workdir, "libdlm_ref_kernels.so")
    cmd = ["nvcc", "-O2", "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
           "-o", so, cu_path]
    subprocess.run(cmd, check=True)
    return ctypes.CDLL(so)


def weights_digest(tensors) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].contiguous().numpy().tobytes())
    return h.hexdigest()


def route_topk(logits: np.ndarray, k: int, norm: bool):
    """src/forward/cpu.rs:980-999 in 32-bit floats."""
    lg = logits.astype(np.float32)
    e = np.exp(lg - lg.max(), dtype=np.float32)
    probs = e / e.sum(dtype=np.float32)
    order = sorted(range(len(probs)), key=lambda i: (-float(probs[i]), i))[:k]
    w = np.array([probs[i] for i in order], dtype=np.float32)
    if norm:
        s = w.sum(dtype=np.float32)
        if s > 0:
            w = w / s
    return [(int(i), float(x)) for i, x in zip(order, w)]


def run_model(lib, raw: dict, tensors: dict, tokens: list[int]) -> np.ndarray:
    """Hidden state after the last layer for every position, [T, H]."""
    dev = torch.device("cuda:0")
    H, nh, L = raw["hidden_size"], raw["num_attention_heads"], raw["num_hidden_layers"]
    nkv = raw.get("num_key_value_heads") or nh
    hd = raw.get("head_dim") or H // nh
    q_dim, kv_dim = nh * hd, nkv * hd
    eps = float(raw["rms_norm_eps"])
    theta = float(raw["rope_theta"])
    E, k = raw.get("num_experts", 0), raw.get("num_experts_per_tok", 0)
    I, Is = raw.get("moe_intermediate_size"), raw.get("shared_expert_intermediate_size")
    inter = raw["intermediate_size"]
    norm = raw.get("norm_topk_prob", True)
    step = raw.get("decoder_sparse_step") or 1
    mlp_only = raw.get("mlp_only_layers") or []

    def d(name):
        return tensors[name].to(torch.float32).contiguous().to(dev)

    def p(t):
        return ctypes.c_void_p(0 if t is None else t.data_ptr())

    W = {n: d(n) for n in tensors}
    inv_freq = torch.tensor([theta ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64) \
        .to(torch.float32).to(dev)                                   # src/forward/cpu.rs:1057-1061
    T = len(tokens)
    keys = [torch.zeros(T * kv_dim, dtype=torch.float32, device=dev) for _ in range(L)]
    values = [torch.zeros(T * kv_dim, dtype=torch.float32, device=dev) for _ in range(L)]
    out = np.zeros((T, H), dtype=np.float32)
    F = ctypes.c_float
    for pos, tok in enumerate(tokens):
        x = W["model.embed_tokens.weight"][tok].clone()
        for i in range(L):
            pre = f"model.layers.{i}."
            attn = [W[pre + f"self_attn.{n}_proj.weight"] for n in "qkvo"]
            bias = [W.get(pre + f"self_attn.{n}_proj.bias") for n in "qkv"]
            ln1, ln2 = W[pre + "input_layernorm.weight"], W[pre + "post_attention_layernorm.weight"]
            sparse = E > 0 and i not in mlp_only and (i + 1) % step == 0
            if not sparse:
                g, u, dn = (W[pre + f"mlp.{n}_proj.weight"] for n in ("gate", "up", "down"))
                rc = lib.dlm_decode_block(H, q_dim, kv_dim, nh, nkv, hd, inter, F(eps), 0, 0,
                                          p(attn[0]), p(attn[1]), p(attn[2]), p(attn[3]), p(g), p(u), p(dn),
                                          p(ln1), p(ln2), p(bias[0]), p(bias[1]), p(bias[2]), p(inv_freq), p(x),
                                          p(keys[i]), p(values[i]), pos, pos)
                assert rc == 0, rc
                continue
            rc = lib.dlm_moe_attn(H, q_dim, kv_dim, nh, nkv, hd, F(eps), 0, 0,
                                  p(attn[0]), p(attn[1]), p(attn[2]), p(attn[3]), p(ln1), p(ln2),
                                  p(bias[0]), p(bias[1]), p(bias[2]), p(inv_freq), p(x),
                                  p(keys[i]), p(values[i]), pos, pos)
            assert rc == 0, rc
            logits = (F * E)()
            rc = lib.dlm_moe_matvec(E, H, 0, 0, p(W[pre + "mlp.gate.weight"]), logits)
            assert rc == 0, rc
            for e, w in route_topk(np.array(list(logits), dtype=np.float32), k, norm):
                g, u, dn = (W[f"{pre}mlp.experts.{e}.{n}_proj.weight"] for n in ("gate", "up", "down"))
                rc = lib.dlm_apply_expert(H, I, 0, 0, p(g), p(u), p(dn), F(w), p(x))
                assert rc == 0, rc
            if Is:
                weight = 1.0
                gate = W.get(pre + "mlp.shared_expert_gate.weight")
                if gate is not None:
                    one = (F * 1)()
                    rc = lib.dlm_moe_matvec(1, H, 0, 0, p(gate), one)
                    assert rc == 0, rc
                    weight = 1.0 / (1.0 + math.exp(-float(np.float32(one[0]))))
                g, u, dn = (W[f"{pre}mlp.shared_expert.{n}_proj.weight"] for n in ("gate", "up", "down"))
                rc = lib.dlm_apply_expert(H, Is, 0, 0, p(g), p(u), p(dn), F(np.float32(weight)), p(x))
                assert rc == 0, rc
        torch.cuda.synchronize()
        out[pos] = x.cpu().numpy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernels-cu", required=True, help="the reference's src/gpu/kernels.cu")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    from safetensors.torch import load_file
    from tiny_configs import TINY, prompt, write_tiny

    with tempfile.TemporaryDirectory() as tmp:
        lib = compile_reference(args.kernels_cu, tmp)
        for fn in ("dlm_decode_block", "dlm_moe_attn", "dlm_moe_matvec", "dlm_apply_expert"):
            getattr(lib, fn).restype = ctypes.c_int
        for name in TINY:
            folder = write_tiny(name, os.path.join(tmp, name))
            raw = json.load(open(os.path.join(folder, "config.json")))
            raw["use_sliding_window"] = False          # the reference has no window
            raw.pop("layer_types", None)
            tensors = load_file(os.path.join(folder, "model.safetensors"))
            tokens = prompt(200, PROMPT_LEN, raw["vocab_size"])
            hidden = run_model(lib, raw, tensors, tokens)
            np.savez(os.path.join(args.out, f"tiny_{name}_reference_kernels.npz"),
                     tokens=np.array(tokens, dtype=np.int32), hidden=hidden,
                     weights_sha256=np.array(weights_digest(tensors)))
            print(f"tiny {name}: hidden {hidden.shape}, |max| {np.abs(hidden).max():.4f}")


if __name__ == "__main__":
    main()
