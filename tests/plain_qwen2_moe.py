"""Plain, slow Qwen2-MoE: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It is written from the reference's
formulas (every function cites the file and lines of vedantnimbarte/dlm it
restates).  The reference's Rust cannot be compiled or imported where these
tests run, but its CUDA model code (src/gpu/kernels.cu) can: outputs of those
kernels on the tiny configurations, made once on a B200 by
``tests/golden/make_golden.py``, are committed under ``tests/golden/`` and
``tests/test_golden.py`` holds this file to them (windows switched off, which
the reference does not have; the window, the tied head and the tie-break rest
on the formulas).  It shares no code with ``dlm_b200``: it reads
``config.json`` with ``json`` and ``model.safetensors`` with the
``safetensors`` package.

Options the reference lacks (a per-layer sliding window, ``decoder_sparse_step``
and ``mlp_only_layers``, ``tie_word_embeddings``) follow the rules stated in
the docstrings below.

``emulate_bf16=True`` rounds to bfloat16 at the places where the engine's
bfloat16 path stores bfloat16 (matrices, normed activations, rotated q/k, v,
attention output, the SwiGLU product); sums, softmax, norms, router logits (taken
from the unrounded normalised residual), rotation angles and the residual stay in
``compute`` precision.
"""
from __future__ import annotations

import json
import math
import os

import torch


# ----------------------------------------------------------------------- loading
def load_folder(path: str):
    """config.json as a dict and every tensor of model.safetensors, by name."""
    from safetensors import safe_open
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    for fn in sorted(os.listdir(path)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(path, fn), framework="pt") as sf:
                for k in sf.keys():
                    tensors[k] = sf.get_tensor(k)
    return cfg, tensors


class PlainConfig:
    """Keys and defaults as src/model/config.rs:425-470 reads them, plus the six keys
    the reference does not read."""

    def __init__(self, raw: dict):
        self.H = raw["hidden_size"]
        self.nh = raw["num_attention_heads"]
        self.nkv = raw.get("num_key_value_heads") or self.nh          # config.rs:444
        self.L = raw["num_hidden_layers"]
        self.V = raw["vocab_size"]
        self.inter = raw.get("intermediate_size") or 4 * self.H       # config.rs:447-449
        self.hd = raw.get("head_dim") or self.H // self.nh            # config.rs:505-508
        self.theta = float(raw.get("rope_theta") or 10000.0)          # config.rs:456
        self.eps = float(raw["rms_norm_eps"]) if raw.get("rms_norm_eps") is not None else 1e-5  # config.rs:457
        self.E = raw.get("num_experts") or 0                          # config.rs:236-243
        self.k = raw.get("num_experts_per_tok") or 0
        self.I = raw.get("moe_intermediate_size") or self.inter       # config.rs:257-264
        self.Is = raw.get("shared_expert_intermediate_size") or None  # config.rs:269
        self.norm_topk = raw.get("norm_topk_prob", True)              # config.rs:271
        if self.norm_topk is None:
            self.norm_topk = True
        self.sparse_step = raw.get("decoder_sparse_step") or 1
        self.mlp_only = list(raw.get("mlp_only_layers") or [])
        self.use_window = bool(raw.get("use_sliding_window") or False)
        self.window = raw.get("sliding_window")
        self.max_window_layers = raw.get("max_window_layers") or 0
        self.layer_types = raw.get("layer_types")
        self.tie = bool(raw.get("tie_word_embeddings") or False)

    def is_sparse(self, i: int) -> bool:
        """Layer i is MoE iff there are experts, i is not in mlp_only_layers and
        (i + 1) % decoder_sparse_step == 0."""
        return self.E > 0 and i not in self.mlp_only and (i + 1) % self.sparse_step == 0

    def layer_window(self, i: int):
        """An explicit layer_types list decides ("sliding_attention" = windowed); without one,
        layer i is windowed iff use_sliding_window and i >= max_window_layers."""
        if self.layer_types is not None:
            return self.window if self.layer_types[i] == "sliding_attention" else None
        return self.window if (self.use_window and i >= self.max_window_layers) else None


# ------------------------------------------------------------------------- parts
def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float32).to(torch.bfloat16).to(x.dtype)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """src/forward/cpu.rs:934-942: mean of squares, inv = 1/sqrt(ms + eps), (v*inv)*w."""
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(ms + eps)
    return (x * inv) * w


def softmax(v: torch.Tensor) -> torch.Tensor:
    """src/forward/cpu.rs:945-957: subtract the max, exp, divide by the sum (last dim)."""
    m = v.max(dim=-1, keepdim=True).values
    e = torch.exp(v - m)
    return e / e.sum(-1, keepdim=True)


def silu(x: torch.Tensor) -> torch.Tensor:
    """src/forward/cpu.rs:960-962: x / (1 + exp(-x))."""
    return x / (1.0 + torch.exp(-x))


def rope_inv_freqs(head_dim: int, theta: float) -> torch.Tensor:
    """src/forward/cpu.rs:1057-1061 without scaling: theta^(-2i/head_dim) as 32-bit floats
    (computed in double and rounded once, so that every platform gets the same table)."""
    return torch.tensor([theta ** (-2.0 * i / head_dim) for i in range(head_dim // 2)],
                        dtype=torch.float64).to(torch.float32)


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """src/forward/cpu.rs:1094-1113: split-half rotation of each head; the angle is the
    32-bit product position * inv_freq.  x: [T, heads, head_dim]."""
    half = x.shape[-1] // 2
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]          # 32-bit product
    sin = torch.sin(ang.to(x.dtype))[:, None, :]
    cos = torch.cos(ang.to(x.dtype))[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window) -> torch.Tensor:
    """src/forward/cpu.rs:1126-1151 for every position at once: query head h reads kv head
    h // (nh / nkv) (:1134), scores scaled by 1/sqrt(head_dim) (:1128), softmax over the
    positions up to the query's own.  With a window W a query at p sees key j iff
    j <= p and p - j < W.  q: [T, nh, hd]; k, v: [T, nkv, hd]."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    pos = torch.arange(T, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= (pos[:, None] - pos[None, :]) < window
    out = torch.zeros_like(q)
    for h in range(nh):
        kvh = h // group
        s = (q[:, h, :] @ k[:, kvh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = softmax(s) @ v[:, kvh, :]
    return out


def swiglu_ffn(x, gate_w, up_w, down_w, rnd):
    """src/forward/cpu.rs:966-971: down · (silu(gate·x) ⊙ up·x)."""
    act = rnd(silu(x @ gate_w.T) * (x @ up_w.T))
    return act @ down_w.T


def route_topk(logits: torch.Tensor, k: int, norm: bool):
    """src/forward/cpu.rs:980-999: softmax over all experts, the k largest probabilities
    (equal probabilities: the lower expert index first), optionally divided by their sum.
    logits: [T, E] -> (ids [T, k], weights [T, k])."""
    probs = softmax(logits)
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :k]
    w = torch.gather(probs, 1, order)
    if norm:
        s = w.sum(-1, keepdim=True)
        w = torch.where(s > 0, w / s, w)
    return order, w


# When a list, moe_ffn appends for every call the gap between the last chosen and the first
# rejected expert's probability at each position (see PlainModel.router_margin).
MARGIN_LOG = None


def moe_ffn(x, lw, cfg: PlainConfig, rnd, x_router=None):
    """src/forward/cpu.rs:1005-1048: routed experts summed from zero in routing order, each
    scaled by its gate weight; then the shared expert scaled by sigmoid(gate·x) (1 when the
    gate tensor is absent)."""
    xr = x if x_router is None else x_router      # the router's input: the unrounded normalised residual
    logits = xr @ lw["router"].T
    ids, wts = route_topk(logits, cfg.k, cfg.norm_topk)
    if MARGIN_LOG is not None and cfg.k < cfg.E:
        sp = torch.sort(softmax(logits), dim=-1, descending=True).values
        MARGIN_LOG.append(sp[:, cfg.k - 1] - sp[:, cfg.k])
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        acc = torch.zeros_like(x[t])
        for j in range(cfg.k):
            e = int(ids[t, j])
            g, u, d = lw["experts"][e]
            acc = acc + wts[t, j] * swiglu_ffn(x[t:t + 1], g, u, d, rnd)[0]
        out[t] = acc
    if lw.get("shared") is not None:
        g, u, d = lw["shared"]
        sh = swiglu_ffn(x, g, u, d, rnd)
        if lw.get("shared_gate") is not None:
            gate = 1.0 / (1.0 + torch.exp(-(xr @ lw["shared_gate"].T)))    # [T, 1]
        else:
            gate = torch.ones(x.shape[0], 1, dtype=x.dtype, device=x.device)
        out = out + gate * sh
    return out


def decoder_layer(x, lw, cfg: PlainConfig, layer_index: int, positions, inv_freq, rnd):
    """src/forward/cpu.rs:1156-1213 for every position at once."""
    T = x.shape[0]
    n = rnd(rmsnorm(x, lw["ln1"], cfg.eps))
    q = n @ lw["q"].T
    k = n @ lw["k"].T
    v = n @ lw["v"].T
    if lw.get("qb") is not None:                       # bias before the rotation (:1177-1179)
        q = q + lw["qb"]
        k = k + lw["kb"]
        v = v + lw["vb"]
    q = rnd(rope(q.view(T, cfg.nh, cfg.hd), positions, inv_freq))
    k = rnd(rope(k.view(T, cfg.nkv, cfg.hd), positions, inv_freq))
    v = rnd(v.view(T, cfg.nkv, cfg.hd))
    ctx = rnd(attention(q, k, v, cfg.layer_window(layer_index)).reshape(T, cfg.nh * cfg.hd))
    x = x + ctx @ lw["o"].T
    n2_full = rmsnorm(x, lw["ln2"], cfg.eps)
    n2 = rnd(n2_full)
    if "router" in lw:
        x = x + moe_ffn(n2, lw, cfg, rnd, x_router=n2_full)
    else:
        g, u, d = lw["dense"]
        x = x + swiglu_ffn(n2, g, u, d, rnd)
    return x


# ------------------------------------------------------------------------- model
class PlainModel:
    def __init__(self, path, compute=torch.float64, emulate_bf16: bool = False, device="cpu"):
        """``path``: a model folder, or a pair (config dict, tensors by name).  ``device``: where the
        plain computation runs (the GPU is only a faster place for the same PyTorch statements)."""
        raw, tensors = path if isinstance(path, tuple) else load_folder(path)
        self.device = torch.device(device)
        self.cfg = cfg = PlainConfig(raw)
        self.compute = compute
        self.rnd = bf16_round if emulate_bf16 else (lambda t: t)

        def mat(name):      # a matrix: rounded to bfloat16 first when that path is emulated
            t = tensors[name].to(self.device).to(torch.float32)
            if emulate_bf16:
                t = t.to(torch.bfloat16).to(torch.float32)
            return t.to(compute)

        def vec(name):      # norm weights and biases keep what they were stored with
            return tensors[name].to(self.device).to(torch.float32).to(compute)

        self.embed = mat("model.embed_tokens.weight")
        self.final_norm = vec("model.norm.weight")
        # src/loader.rs:711-715: no lm_head.weight -> the embedding serves as head
        if cfg.tie or "lm_head.weight" not in tensors:
            self.lm_head = self.embed
        else:
            self.lm_head = mat("lm_head.weight")
        self.layers = []
        for i in range(cfg.L):
            p = f"model.layers.{i}."
            lw = {"ln1": vec(p + "input_layernorm.weight"), "ln2": vec(p + "post_attention_layernorm.weight"),
                  "q": mat(p + "self_attn.q_proj.weight"), "k": mat(p + "self_attn.k_proj.weight"),
                  "v": mat(p + "self_attn.v_proj.weight"), "o": mat(p + "self_attn.o_proj.weight")}
            if p + "self_attn.q_proj.bias" in tensors:      # src/loader.rs:258-264, 415-417
                lw["qb"] = vec(p + "self_attn.q_proj.bias")
                lw["kb"] = vec(p + "self_attn.k_proj.bias")
                lw["vb"] = vec(p + "self_attn.v_proj.bias")
            if cfg.is_sparse(i):                            # names: src/loader.rs:434-453
                lw["router"] = mat(p + "mlp.gate.weight")
                lw["experts"] = [tuple(mat(f"{p}mlp.experts.{e}.{n}_proj.weight") for n in ("gate", "up", "down"))
                                 for e in range(cfg.E)]
                if cfg.Is:
                    lw["shared"] = tuple(mat(f"{p}mlp.shared_expert.{n}_proj.weight") for n in ("gate", "up", "down"))
                    if p + "mlp.shared_expert_gate.weight" in tensors:
                        lw["shared_gate"] = mat(p + "mlp.shared_expert_gate.weight")
            else:                                           # src/loader.rs:395-399
                lw["dense"] = tuple(mat(f"{p}mlp.{n}_proj.weight") for n in ("gate", "up", "down"))
            self.layers.append(lw)
        self.inv_freq = rope_inv_freqs(cfg.hd, cfg.theta).to(self.device)

    def hidden_states(self, tokens, layer_order=None) -> torch.Tensor:
        """Residual stream after the last layer for the whole sequence [T, H]."""
        cfg = self.cfg
        ids = torch.as_tensor(tokens, dtype=torch.long)
        if ids.numel() == 0 or int(ids.max()) >= cfg.V or int(ids.min()) < 0:
            raise ValueError("empty prompt or token outside the vocabulary")   # src/generate.rs:315-325
        ids = ids.to(self.device)
        x = self.embed[ids]                                  # row copy, no scaling
        positions = torch.arange(ids.numel(), device=self.device)
        order = range(cfg.L) if layer_order is None else layer_order
        for i in order:
            x = decoder_layer(x, self.layers[i], cfg, i, positions, self.inv_freq, self.rnd)
        return x

    def router_margins(self, tokens) -> torch.Tensor:
        """For every position, the smallest gap over the routed layers between the probability
        of the last expert chosen and the first one rejected.  Top-k is discontinuous: where
        this gap is within rounding, two correct implementations may route differently; tests
        do not compare such positions."""
        global MARGIN_LOG
        MARGIN_LOG = []
        try:
            self.hidden_states(tokens)
            gaps = list(MARGIN_LOG)
        finally:
            MARGIN_LOG = None
        if not gaps:
            return torch.full((len(tokens),), float("inf"), dtype=torch.float64)
        return torch.stack([g.to(torch.float64) for g in gaps]).min(dim=0).values.cpu()

    def logits(self, tokens, layer_order=None) -> torch.Tensor:
        """src/generate.rs:328-331 at every position: rmsnorm with model.norm, then the head.
        Returns [T, V] as 32-bit floats."""
        x = self.hidden_states(tokens, layer_order)
        n = self.rnd(rmsnorm(x, self.final_norm, self.cfg.eps))
        return (n @ self.lm_head.T).to(torch.float32).cpu()


# ---------------------------------------------------------------------- sampling
class SplitMix64:
    """src/generate.rs:37-57."""
    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.s = (seed ^ 0x9E3779B97F4A7C15) & self.MASK

    def next_u64(self) -> int:
        self.s = (self.s + 0x9E3779B97F4A7C15) & self.MASK
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self.MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self.MASK
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


def argmax(logits) -> int:
    """src/generate.rs:22-32: the first maximum wins."""
    best, best_val = 0, float("-inf")
    for i, v in enumerate(logits.tolist()):
        if v > best_val:
            best, best_val = i, v
    return best


def apply_repetition_penalty(logits: torch.Tensor, seen, penalty: float) -> torch.Tensor:
    """src/generate.rs:122-132: seen tokens' logits divided by the penalty when positive,
    multiplied when not."""
    if penalty == 1.0:
        return logits
    out = logits.clone()
    for t in set(int(s) for s in seen):
        if t < out.numel():
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def sample_topk_topp(logits: torch.Tensor, temperature: float, top_p: float, top_k: int, min_p: float,
                     rng: SplitMix64) -> int:
    """src/generate.rs:136-210, in 32-bit floats as there.  Equal logits: lower index first."""
    f32 = torch.float32
    lg = logits.to(f32)
    idx = torch.sort(lg, descending=True, stable=True).indices
    k = min(top_k, idx.numel()) if top_k > 0 else idx.numel()
    idx = idx[:k]
    mx = lg[idx[0]]
    probs = torch.exp((lg[idx] - mx) / torch.tensor(temperature, dtype=f32))
    probs = probs / probs.sum()
    if 0.0 < top_p < 1.0:
        cum = torch.cumsum(probs, 0)
        hit = torch.nonzero(cum >= top_p)
        cut = int(hit[0]) + 1 if hit.numel() else probs.numel()
        probs, idx = probs[:cut], idx[:cut]
        probs = probs / probs.sum()
    if min_p > 0.0:
        thr = min_p * probs[0]
        keep = 0
        for p in probs.tolist():
            if p >= float(thr):
                keep += 1
            else:
                break
        keep = max(keep, 1)
        probs, idx = probs[:keep], idx[:keep]
        probs = probs / probs.sum()
    r = rng.next_f32()
    cum = torch.cumsum(probs, 0)
    hit = torch.nonzero(cum > r)
    return int(idx[int(hit[0])]) if hit.numel() else int(idx[-1])


def generate(model: PlainModel, prompt, max_new_tokens=16, eos_token=None, temperature=0.0, top_p=1.0,
             top_k=0, min_p=0.0, repetition_penalty=1.0, seed=0):
    """src/generate.rs:338-373 without a cache: the whole sequence is run again for every
    token.  The end-of-sequence token is part of the output (:364-368)."""
    tokens = list(prompt)
    rng = SplitMix64(seed)
    out = []
    for _ in range(max_new_tokens):
        lg = model.logits(tokens)[-1]
        lg = apply_repetition_penalty(lg, tokens, repetition_penalty)
        if temperature <= 0.0:
            nxt = argmax(lg)
        else:
            nxt = sample_topk_topp(lg, temperature, top_p, top_k, min_p, rng)
        out.append(nxt)
        tokens.append(nxt)
        if eos_token is not None and nxt == eos_token:
            break
    return out
