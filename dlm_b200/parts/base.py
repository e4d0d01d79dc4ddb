"""Interfaces of the parts a model is put together from.

A *part* has its sizes and constants as constructor parameters and never
learns which model it is in.  It names its tensors relative to itself
(``q_proj.weight``); the model prefixes them.  Four kinds of part exist:

* ``Norm``              ``forward(x_f32, rt, rows=None) -> activations``
* ``PositionEncoding``  gives the rotation table the attention kernels apply
* ``Mixer``             ``forward(h, resid, ctx, call)``: adds its output to ``resid``
* ``FeedForward``       ``forward(h, resid, ctx, pre_norm)``: adds its output to ``resid``

and a ``Block`` arranges one mixer, one feed-forward and their norms.

The residual stream ``resid`` is always 32-bit; ``h`` has the runtime's
activation dtype.  A mixer states what it needs cached through
``cache_need()`` (paged keys and values) and ``state_need()`` (a tensor of
fixed size per request); the cache manager groups equal needs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part reads.  ``init`` says how the random-weights mode draws it:
    ``linear`` N(0, 0.02), ``bias`` N(0, 0.02), ``norm`` 1 + N(0, 0.02)."""
    name: str
    shape: tuple[int, ...]
    init: str = "linear"
    optional: bool = False


@dataclass(frozen=True)
class PagedKV:
    """A mixer's need for cached keys and values: per token ``num_kv_heads * head_dim``
    keys and as many values; ``window`` None keeps all of them, W keeps the last W."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class RequestState:
    """A mixer's need for a tensor of fixed size per request (zeroed when a request starts)."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class PartSpec:
    """Which part to build (a name in the registry of its kind) and its parameters."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)


class Runtime:
    """Device, activation dtype and the kernel backend, handed to every part."""

    def __init__(self, device, dtype: torch.dtype, ops):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype
        self.ops = ops

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A weight matrix in the activation dtype on the device."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights and biases: always 32-bit (they enter 32-bit arithmetic)."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()


class Part:
    def param_specs(self) -> list[ParamSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        """``tensors`` maps this part's relative names to the stored tensors (optional ones
        may be absent)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, rt: Runtime, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """``rotary()`` returns None or ``(inv_freq f32[rotary_dim/2] on the device, rotary_dim)``:
    dimension pairs ``(i, i + rotary_dim/2)`` of each head are rotated by
    ``position * inv_freq[i]``; dimensions from ``rotary_dim`` on pass through."""

    def rotary(self, rt: Runtime):
        return None

    def on_embed(self, x: torch.Tensor, positions: torch.Tensor, rt: Runtime) -> None:
        """Hook for encodings that act on the embedded tokens (in place); default: nothing."""


class Mixer(Part):
    def cache_need(self) -> PagedKV | None:
        return None

    def state_need(self) -> RequestState | None:
        return None

    def forward(self, h: torch.Tensor, resid: torch.Tensor, ctx: "StepContext", call: int) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, resid: torch.Tensor, ctx: "StepContext", pre_norm: "Norm | None" = None) -> None:
        """``pre_norm`` is the norm that produced ``h`` from ``resid``; a part that needs the
        normalised input in 32-bit (a router) may apply it again to the residual itself."""
        raise NotImplementedError


@dataclass
class GroupView:
    """What one cache group contributes to a step: where the new tokens' keys and values go
    and each request's block table."""
    slots: torch.Tensor         # i32 [T]   page * page_size + offset
    block_table: torch.Tensor   # i32 [R, width]
    page_size: int
    window: int                 # 0: none


@dataclass
class StepBatch:
    """Device-side description of one step: a flat array of tokens of several requests."""
    num_tokens: int
    num_requests: int
    tokens: torch.Tensor        # i32 [T]
    positions: torch.Tensor     # i32 [T]  absolute position of each token in its request
    token_req: torch.Tensor     # i32 [T]  row of the request each token belongs to
    cu_q: torch.Tensor          # i32 [R+1] start of each request's tokens
    kv_len: torch.Tensor        # i32 [R]  tokens the request holds after this step
    state_slot: torch.Tensor    # i32 [R]  the request's state slot
    logit_rows: torch.Tensor    # i32 [N]  flat places whose logits are wanted
    groups: list[GroupView]
    max_q_len: int
    max_kv_len: int
    num_single: int = 0         # requests with exactly one token in this step


@dataclass
class PagedView:
    k: torch.Tensor             # [pages, num_kv_heads, page_size, head_dim]
    v: torch.Tensor
    group: GroupView
    write: bool                 # False when this call only reads another call's cache


class StepContext:
    """What a mixer or feed-forward may ask for during a step."""

    def __init__(self, rt: Runtime, batch: StepBatch, paged_of_call: Callable[[int], PagedView | None],
                 state_of_call: Callable[[int], torch.Tensor | None]):
        self.rt = rt
        self.batch = batch
        self._paged = paged_of_call
        self._state = state_of_call

    def paged(self, call: int) -> PagedView:
        v = self._paged(call)
        if v is None:
            raise RuntimeError(f"layer call {call} asked for paged keys/values but declared no need for them")
        return v

    def state(self, call: int) -> torch.Tensor:
        s = self._state(call)
        if s is None:
            raise RuntimeError(f"layer call {call} asked for per-request state but declared no need for it")
        return s
