"""How a mixer, a feed-forward and their norms are arranged in one layer."""
from __future__ import annotations

from ..registry import build_part, register_part
from .base import Part, PartSpec, StepContext


class PreNormBlock(Part):
    """``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/forward/cpu.rs:1171-1212).  The
    residual ``x`` stays 32-bit; each sub-part adds into it."""

    # sub-part -> name prefix inside the layer
    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec,
                 names: dict[str, str] | None = None):
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.norm2 = build_part("norm", norm2)
        self.ffn = build_part("ffn", ffn)
        self.names = {"norm1": "norm1.", "mixer": "mixer.", "norm2": "norm2.", "ffn": "ffn."}
        if names:
            self.names.update(names)

    def children(self):
        return [(self.names["norm1"], self.norm1), (self.names["mixer"], self.mixer),
                (self.names["norm2"], self.norm2), (self.names["ffn"], self.ffn)]

    def param_specs(self):
        out = []
        for prefix, part in self.children():
            for s in part.param_specs():
                out.append(type(s)(prefix + s.name, s.shape, s.init, s.optional))
        return out

    def load(self, tensors, rt):
        for prefix, part in self.children():
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, rt)

    def forward(self, resid, ctx: StepContext, call: int):
        rt = ctx.rt
        self.mixer.forward(self.norm1.forward(resid, rt), resid, ctx, call)
        self.ffn.forward(self.norm2.forward(resid, rt), resid, ctx, pre_norm=self.norm2)


register_part("block", "prenorm", PreNormBlock)
