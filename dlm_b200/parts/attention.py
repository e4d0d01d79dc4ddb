"""Attention mixers."""
from __future__ import annotations

import math

import torch

from ..registry import build_part, register_part
from .base import Mixer, PagedKV, ParamSpec, PartSpec, Runtime, StepContext


class GroupedQueryAttention(Mixer):
    """Softmax attention over paged keys and values with grouped query heads
    (src/forward/cpu.rs:1171-1193, 1126-1151): q/k/v projections (bias optional, added
    before the rotation), position encoding on q and k, keys stored rotated, query head h
    reads kv head ``h // (heads / kv_heads)``, scores scaled by ``1/sqrt(head_dim)``,
    output projection without bias added to the residual.  With ``window`` W a query at
    position p sees key j iff ``j <= p`` and ``p - j < W``.

    The three projections are concatenated at load into one ``[Q + 2KV, hidden]`` matrix.
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool | None = None, window: int | None = None,
                 position: PartSpec | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.qkv_bias = qkv_bias          # None: decided by the presence of the bias tensors
        self.window = int(window) if window else None
        self.position = build_part("position", position) if position is not None else None
        self.q_dim, self.kv_dim = self.nh * self.hd, self.nkv * self.hd
        self.scale = 1.0 / math.sqrt(self.hd)
        self.w_qkv = self.b_qkv = self.w_o = None

    def param_specs(self):
        opt = self.qkv_bias is None
        specs = [ParamSpec("q_proj.weight", (self.q_dim, self.hidden)),
                 ParamSpec("k_proj.weight", (self.kv_dim, self.hidden)),
                 ParamSpec("v_proj.weight", (self.kv_dim, self.hidden)),
                 ParamSpec("o_proj.weight", (self.hidden, self.q_dim))]
        if self.qkv_bias is not False:
            specs += [ParamSpec("q_proj.bias", (self.q_dim,), init="bias", optional=opt),
                      ParamSpec("k_proj.bias", (self.kv_dim,), init="bias", optional=opt),
                      ParamSpec("v_proj.bias", (self.kv_dim,), init="bias", optional=opt)]
        return specs

    def load(self, tensors, rt: Runtime):
        self.w_qkv = torch.cat([rt.matrix(tensors[f"{n}_proj.weight"]) for n in "qkv"], dim=0).contiguous()
        self.w_o = rt.matrix(tensors["o_proj.weight"])
        have = [f"{n}_proj.bias" in tensors for n in "qkv"]
        if any(have):
            parts = []
            for n, size in zip("qkv", (self.q_dim, self.kv_dim, self.kv_dim)):
                key = f"{n}_proj.bias"
                parts.append(rt.vector(tensors[key]) if key in tensors
                             else torch.zeros(size, dtype=torch.float32, device=rt.device))
            self.b_qkv = torch.cat(parts).contiguous()
        else:
            self.b_qkv = None

    def cache_need(self):
        return PagedKV(self.nkv, self.hd, self.window)

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        view = ctx.paged(call)
        qkv = ops.linear(h, self.w_qkv, self.b_qkv, torch.float32)
        rot = self.position.rotary(rt) if self.position is not None else None
        inv_freq, rotary_dim = rot if rot is not None else (None, 0)
        q = ops.rope_kv_write(qkv, b.positions, inv_freq, rotary_dim,
                              view.group.slots if view.write else None,
                              view.k, view.v, self.nh, self.nkv, self.hd, rt.dtype,
                              interleaved=bool(rot is not None and self.position.interleaved))
        o = ops.attention(q, view.k, view.v, view.group.block_table, b.cu_q, b.kv_len,
                          self.window or 0, self.scale, self.nh, self.nkv, self.hd,
                          b.max_q_len, b.max_kv_len, b.num_single)
        ops.linear_add(o, self.w_o, resid)


register_part("mixer", "gqa_attention", GroupedQueryAttention)
