"""Choosing the next token: the reference's samplers (src/generate.rs:61-210) on the device.

``SamplingParams`` carries the reference's options with its names and defaults.  The
uniform numbers come from a per-request SplitMix64 on the host (one draw per sampled
token, as ``Sampler::sample`` makes); everything over the vocabulary runs in the
sampling kernels.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

_MASK = (1 << 64) - 1


class SplitMix64:
    """src/generate.rs:37-57: state ``seed ^ 0x9E37..7C15``; ``next_f32`` is the top 24 bits / 2^24."""

    def __init__(self, seed: int):
        self.state = (int(seed) ^ 0x9E3779B97F4A7C15) & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


@dataclass
class SamplingParams:
    """``temperature <= 0`` is greedy (the first maximum wins); ``top_k == 0`` keeps every
    token; ``top_p >= 1`` or ``<= 0`` disables the nucleus cut; ``min_p <= 0`` disables
    min-p; ``repetition_penalty == 1`` disables the penalty (src/generate.rs:61-81)."""
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)

    @property
    def plain_greedy(self) -> bool:
        return self.greedy and self.repetition_penalty == 1.0


class RequestSampler:
    """Per-request sampling state: the generator and the set of tokens seen so far."""

    def __init__(self, params: SamplingParams, prompt):
        self.params = params
        self.rng = SplitMix64(params.seed)
        self.seen: dict[int, None] = dict.fromkeys(int(t) for t in prompt) if params.repetition_penalty != 1.0 else {}

    def note(self, token: int) -> None:
        if self.params.repetition_penalty != 1.0:
            self.seen[int(token)] = None


def sample_rows(ops, logits: torch.Tensor, samplers: list[RequestSampler]) -> list[int]:
    """One token per row of ``logits`` ([N, V], 32-bit, on the device).  Advances each
    non-greedy request's generator by one draw."""
    n = logits.shape[0]
    if n == 0:
        return []
    if all(s.params.plain_greedy for s in samplers):
        return ops.argmax(logits).tolist()
    dev = logits.device
    params = torch.tensor([[s.params.temperature, s.params.top_p, s.params.min_p, s.params.repetition_penalty]
                           for s in samplers], dtype=torch.float32)
    top_k = torch.tensor([s.params.top_k for s in samplers], dtype=torch.int32)
    u = torch.tensor([0.0 if s.params.greedy else s.rng.next_f32() for s in samplers], dtype=torch.float32)
    offsets, seen = [0], []
    for s in samplers:
        seen.extend(s.seen.keys())
        offsets.append(len(seen))
    seen_offsets = torch.tensor(offsets, dtype=torch.int32)
    seen_tokens = torch.tensor(seen if seen else [0], dtype=torch.int32)
    out = ops.sample(logits, params.to(dev), top_k.to(dev), u.to(dev), seen_offsets.to(dev), seen_tokens.to(dev))
    return out.tolist()
