"""Interfaces of the parts a model is put together from.

A *part* has its sizes and constants as constructor parameters and never
learns which model it is in.  It names its tensors relative to itself
(``q_proj.weight``); the model prefixes them.  Four kinds of part exist:

* ``Norm``              ``forward(x_f32, rt, rows=None, out_dtype=None) -> activations``
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
class CacheTensor:
    """One paged tensor of a mixer's cache: per token ``heads`` rows of ``width`` elements,
    laid out ``[pages, heads, page_size, width]``."""
    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class PagedCache:
    """What a mixer wants cached per token, in pages: any number of tensors (keys and values, or
    one latent vector, ...).  ``window`` None keeps every token, W keeps the last W (older pages go
    back to the pool).  ``page_size`` None takes the engine's page size; layers whose window and
    page size agree share a pool of pages and a block table."""
    tensors: tuple[CacheTensor, ...]
    window: int | None = None
    page_size: int | None = None

    def elements_per_token(self) -> int:
        return sum(t.heads * t.width for t in self.tensors)

    def same_layout(self, other: "PagedCache") -> bool:
        return self.tensors == other.tensors and self.page_size == other.page_size


def PagedKV(num_kv_heads: int, head_dim: int, window: int | None = None, page_size: int | None = None) -> PagedCache:
    """The need of an attention mixer: per token ``num_kv_heads * head_dim`` keys (tensor ``k``)
    and as many values (tensor ``v``)."""
    return PagedCache((CacheTensor("k", int(num_kv_heads), int(head_dim)),
                       CacheTensor("v", int(num_kv_heads), int(head_dim))), window, page_size)


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
    # False for a part whose forward reads device data on the host (a synchronisation): steps of a
    # model that holds one are not captured in CUDA graphs.
    graph_safe = True

    def param_specs(self) -> list[ParamSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        """``tensors`` maps this part's relative names to the stored tensors (optional ones
        may be absent)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, rt: Runtime, rows: torch.Tensor | None = None,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """Normalises the 32-bit rows ``x`` (only ``rows`` of them when given); the result has
        ``out_dtype``, the runtime's activation dtype when None."""
        raise NotImplementedError

    def fusable_rms(self) -> tuple[torch.Tensor, float] | None:
        """``(weight, eps)`` if this norm is a plain RMS norm that a kernel may apply itself to the
        32-bit residual (the router's kernel does), else None: the caller then asks ``forward`` for a
        32-bit result."""
        return None


class PositionEncoding(Part):
    """``rotary()`` returns None or ``(inv_freq f32[rotary_dim/2] on the device, rotary_dim)``:
    pair i of each head is rotated by ``position * inv_freq[i]``; dimensions from ``rotary_dim``
    on pass through.  Pair i is dims ``(i, i + rotary_dim/2)``, or ``(2i, 2i + 1)`` when the
    class attribute ``interleaved`` is True."""

    interleaved = False

    def rotary(self, rt: Runtime):
        return None

    def on_embed(self, x: torch.Tensor, positions: torch.Tensor, rt: Runtime) -> None:
        """Hook for encodings that act on the embedded tokens (in place); default: nothing."""


class Mixer(Part):
    def cache_need(self) -> PagedCache | None:
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
    tensors: dict[str, torch.Tensor]   # by CacheTensor.name: [pages, heads, page_size, width]
    group: GroupView
    write: bool                 # False when this call only reads another call's cache

    @property
    def k(self) -> torch.Tensor:
        return self.tensors["k"]

    @property
    def v(self) -> torch.Tensor:
        return self.tensors["v"]


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
