"""A decoder model put together from parts according to a ``ModelSpec``.

The spec is data: which block each layer is, which tensors' names it reads, and
the *order* in which layers run.  The order is a list of ``LayerCall``; it may
name a layer twice, and a call may read the cache an earlier call wrote instead
of writing one of its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..registry import build_part
from .base import PagedView, ParamSpec, PartSpec, Runtime, StepBatch, StepContext


@dataclass(frozen=True)
class LayerCall:
    layer: int
    reads_cache_of: int | None = None   # index (in the order) of an earlier call whose cache is read


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: list[PartSpec]               # block specs
    layer_prefixes: list[str]            # tensor-name prefix of each layer ("model.layers.0.")
    final_norm: PartSpec
    final_norm_prefix: str = "model.norm."
    embed_name: str = "model.embed_tokens.weight"
    lm_head_name: str = "lm_head.weight"
    tie_word_embeddings: bool = False    # True: the embedding is the head; False: tied iff the head is absent
    order: list[LayerCall] | None = None # None: every layer once, in index order
    embed_position: PartSpec | None = None   # a position encoding that acts on the embedded tokens


class WeightError(ValueError):
    """Lists, in one message, every missing tensor, unexpected tensor and wrong shape."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["the checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing[:40])
                         + (" ..." if len(self.missing) > 40 else ""))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected[:40])
                         + (" ..." if len(self.unexpected) > 40 else ""))
        for name, got, want in self.wrong_shape[:40]:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype[:40]:
            lines.append(f"  unsupported dtype: {name} is {got}")
        super().__init__("\n".join(lines))


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec, self.rt = spec, rt
        self.blocks = [build_part("block", bs) for bs in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.embed_position = build_part("position", spec.embed_position) if spec.embed_position else None
        self.order = list(spec.order) if spec.order is not None else [LayerCall(i) for i in range(len(self.blocks))]
        for ci, c in enumerate(self.order):
            if not (0 <= c.layer < len(self.blocks)):
                raise ValueError(f"order names layer {c.layer}, the model has {len(self.blocks)}")
            if c.reads_cache_of is not None:
                if not (0 <= c.reads_cache_of < ci) or self.order[c.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"call {ci} must read the cache of an earlier call that owns one")
                a = self.blocks[c.layer].mixer.cache_need()
                b = self.blocks[self.order[c.reads_cache_of].layer].mixer.cache_need()
                if a is None or b is None or not a.same_layout(b):
                    raise ValueError(f"call {ci} cannot read call {c.reads_cache_of}'s cache: their shapes differ")
        self.embed: torch.Tensor | None = None
        self.lm_head: torch.Tensor | None = None

    # ------------------------------------------------------------- tensors
    def param_specs(self) -> dict[str, ParamSpec]:
        s = self.spec
        out = {s.embed_name: ParamSpec(s.embed_name, (s.vocab_size, s.hidden_size))}
        for prefix, block in zip(s.layer_prefixes, self.blocks):
            for p in block.param_specs():
                out[prefix + p.name] = ParamSpec(prefix + p.name, p.shape, p.init, p.optional)
        for p in self.final_norm.param_specs():
            out[s.final_norm_prefix + p.name] = ParamSpec(s.final_norm_prefix + p.name, p.shape, p.init, p.optional)
        out[s.lm_head_name] = ParamSpec(s.lm_head_name, (s.vocab_size, s.hidden_size), optional=True)
        return out

    def check(self, available: dict[str, tuple[torch.dtype, tuple[int, ...]]]) -> None:
        """Raises ``WeightError`` unless ``available`` (name -> dtype, shape) fits the model."""
        specs = self.param_specs()
        missing = [n for n, p in specs.items() if not p.optional and n not in available]
        unexpected = [n for n in available if n not in specs]
        wrong, wrong_dt = [], []
        for n, (dt, shape) in available.items():
            if n in specs:
                if tuple(shape) != tuple(specs[n].shape):
                    wrong.append((n, shape, specs[n].shape))
                if dt not in (torch.float32, torch.bfloat16, torch.float16, torch.float64):
                    wrong_dt.append((n, dt))
        if missing or unexpected or wrong or wrong_dt:
            raise WeightError(sorted(missing), sorted(unexpected), wrong, wrong_dt)

    def load(self, get, names) -> None:
        """``get(name) -> tensor`` for every name in ``names`` (already checked)."""
        s, rt = self.spec, self.rt
        names = set(names)
        self.embed = rt.matrix(get(s.embed_name))
        if s.tie_word_embeddings or s.lm_head_name not in names:
            self.lm_head = self.embed                  # an alias, not a copy
        else:
            self.lm_head = rt.matrix(get(s.lm_head_name))
        for prefix, block in zip(s.layer_prefixes, self.blocks):
            block.load({n[len(prefix):]: get(n) for n in names if n.startswith(prefix)}, rt)
        self.final_norm.load({n[len(s.final_norm_prefix):]: get(n) for n in names
                              if n.startswith(s.final_norm_prefix)}, rt)

    # --------------------------------------------------------------- cache
    def cache_needs(self):
        """Per call of the order: (PagedCache or None, RequestState or None, owner call index)."""
        out = []
        for ci, c in enumerate(self.order):
            mixer = self.blocks[c.layer].mixer
            owner = ci if c.reads_cache_of is None else c.reads_cache_of
            out.append((mixer.cache_need(), mixer.state_need(), owner))
        return out

    # ---------------------------------------------------------------- step
    def step(self, batch: StepBatch, cache) -> torch.Tensor:
        """Runs the batch's tokens through every call of the order, reading and writing
        ``cache``; returns 32-bit logits ``[len(batch.logit_rows), vocab]``."""
        rt, ops = self.rt, self.rt.ops

        def paged(call):
            return cache.paged_view(call, batch)

        ctx = StepContext(rt, batch, paged, cache.state_tensor)
        x = ops.embed(batch.tokens, self.embed)
        if self.embed_position is not None:
            self.embed_position.on_embed(x, batch.positions, rt)
        for ci, c in enumerate(self.order):
            self.blocks[c.layer].forward(x, ctx, ci)
        n = self.final_norm.forward(x, rt, rows=batch.logit_rows)
        return ops.linear(n, self.lm_head, None, torch.float32)
