"""Feed-forward parts: a dense SwiGLU MLP and a routed mixture of SwiGLU experts."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import FeedForward, ParamSpec, Runtime, StepContext


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows ``2i`` = gate row i, ``2i + 1`` = up row i, so that a SwiGLU epilogue finds both
    halves of an output in neighbouring accumulator columns."""
    out = torch.empty((2 * gate.shape[0], gate.shape[1]), dtype=gate.dtype, device=gate.device)
    out[0::2] = gate
    out[1::2] = up
    return out


class DenseSwiGLU(FeedForward):
    """``resid += down · (silu(gate·h) ⊙ up·h)`` without biases (src/forward/cpu.rs:966-971, 1198)."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def param_specs(self):
        return [ParamSpec("gate_proj.weight", (self.inter, self.hidden)),
                ParamSpec("up_proj.weight", (self.inter, self.hidden)),
                ParamSpec("down_proj.weight", (self.hidden, self.inter))]

    def load(self, tensors, rt: Runtime):
        self.w_gate_up = interleave_gate_up(rt.matrix(tensors["gate_proj.weight"]), rt.matrix(tensors["up_proj.weight"]))
        self.w_down = rt.matrix(tensors["down_proj.weight"])

    def forward(self, h, resid, ctx: StepContext, pre_norm=None):
        ops = ctx.rt.ops
        act = ops.linear_swiglu(h, self.w_gate_up)
        ops.linear_add(act, self.w_down, resid)


class SoftmaxTopKMoE(FeedForward):
    """Routed experts as the reference computes them (src/forward/cpu.rs:980-1048): router
    logits in 32-bit from the 32-bit normalised residual, softmax over all experts, the k largest probabilities (ties: lower
    expert first), optionally renormalised; each chosen expert's SwiGLU output scaled by its
    weight and summed from zero in routing order; then an optional shared expert scaled by
    ``sigmoid(shared_gate · h)``; the sum goes to the residual.  ``shared_gate``: True, the gate
    tensor is required; False, there is none and the factor is 1; None, the checkpoint decides:
    a missing gate tensor means the factor 1 (src/forward/cpu.rs:1032-1041).

    At load the experts are stacked into ``[E, 2I, H]`` (gate and up rows interleaved) and
    ``[E, H, I]``; the router and the shared gate become one ``[E (+1), H]`` matrix."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, expert_intermediate_size: int,
                 norm_topk_prob: bool, shared_intermediate_size: int | None = None,
                 shared_gate: bool | None = True):
        self.hidden, self.E, self.k, self.I = int(hidden_size), int(num_experts), int(top_k), int(expert_intermediate_size)
        if not (1 <= self.k <= self.E):
            raise ValueError("top_k must be in 1..num_experts")
        self.norm = bool(norm_topk_prob)
        self.Is = int(shared_intermediate_size) if shared_intermediate_size else None
        self.shared_gate = shared_gate if self.Is is not None else False
        self.has_gate = bool(self.shared_gate)      # None: settled when the tensors are loaded
        self.w_router = self.w_gate_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def param_specs(self):
        specs = [ParamSpec("gate.weight", (self.E, self.hidden))]
        for e in range(self.E):
            specs += [ParamSpec(f"experts.{e}.gate_proj.weight", (self.I, self.hidden)),
                      ParamSpec(f"experts.{e}.up_proj.weight", (self.I, self.hidden)),
                      ParamSpec(f"experts.{e}.down_proj.weight", (self.hidden, self.I))]
        if self.Is:
            specs += [ParamSpec("shared_expert.gate_proj.weight", (self.Is, self.hidden)),
                      ParamSpec("shared_expert.up_proj.weight", (self.Is, self.hidden)),
                      ParamSpec("shared_expert.down_proj.weight", (self.hidden, self.Is))]
            if self.shared_gate is not False:
                specs.append(ParamSpec("shared_expert_gate.weight", (1, self.hidden),
                                       optional=self.shared_gate is None))
        return specs

    def load(self, tensors, rt: Runtime):
        rows = [rt.matrix(tensors["gate.weight"])]
        self.has_gate = (self.shared_gate is True
                         or (self.shared_gate is None and "shared_expert_gate.weight" in tensors))
        if self.has_gate:
            rows.append(rt.matrix(tensors["shared_expert_gate.weight"]).reshape(1, self.hidden))
        self.w_router = torch.cat(rows, dim=0).contiguous()
        self.w_gate_up = torch.empty((self.E, 2 * self.I, self.hidden), dtype=rt.dtype, device=rt.device)
        self.w_down = torch.empty((self.E, self.hidden, self.I), dtype=rt.dtype, device=rt.device)
        for e in range(self.E):
            self.w_gate_up[e, 0::2] = rt.matrix(tensors[f"experts.{e}.gate_proj.weight"])
            self.w_gate_up[e, 1::2] = rt.matrix(tensors[f"experts.{e}.up_proj.weight"])
            self.w_down[e] = rt.matrix(tensors[f"experts.{e}.down_proj.weight"])
        if self.Is:
            self.ws_gate_up = interleave_gate_up(rt.matrix(tensors["shared_expert.gate_proj.weight"]),
                                                 rt.matrix(tensors["shared_expert.up_proj.weight"]))
            self.ws_down = rt.matrix(tensors["shared_expert.down_proj.weight"])

    def forward(self, h, resid, ctx: StepContext, pre_norm=None):
        ops = ctx.rt.ops
        rms = pre_norm.fusable_rms() if pre_norm is not None else None
        shared = None
        branch = ops.branch(h.shape[0])
        if self.Is:
            # the shared expert needs nothing from the router: it may run beside the routed experts
            with branch:
                sact = ops.linear_swiglu(h, self.ws_gate_up)
                shared = ops.linear(sact, self.ws_down, None, torch.float32)
        # router logits (and the shared expert's gate) from the 32-bit normalised residual: an RMS norm is
        # applied again inside the router's kernel, any other norm is asked for a 32-bit result
        if rms is not None:
            # (the residual was last written before ``pre_norm`` ran: the kernel launched just before this
            # one, the norm's or the shared expert's, only reads it)
            ids, wts, gate, offsets, rows, dest = ops.route(resid, self.w_router, self.E, self.k, self.norm,
                                                            self.has_gate, norm_weight=rms[0], eps=rms[1],
                                                            input_settled=True)
        else:
            x = h if pre_norm is None else pre_norm.forward(resid, ctx.rt, out_dtype=torch.float32)
            ids, wts, gate, offsets, rows, dest = ops.route(x, self.w_router, self.E, self.k, self.norm, self.has_gate)
        act = ops.grouped_swiglu(h, self.w_gate_up, offsets, rows)
        y = ops.grouped_linear(act, self.w_down, offsets)
        branch.join()
        ops.moe_combine(y, dest, wts, shared, gate, resid)


register_part("ffn", "swiglu_dense", DenseSwiGLU)
register_part("ffn", "moe_softmax_topk", SoftmaxTopKMoE)
