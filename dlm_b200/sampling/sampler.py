"""Choosing the next token: the reference's samplers (src/generate.rs:61-210) on the device.

``SamplingParams`` carries the reference's options with its names and defaults.  The
uniform numbers come from a per-request SplitMix64 on the host (one draw per sampled
token, as ``Sampler::sample`` makes); everything over the vocabulary runs in the
sampling kernels.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
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
    """Per-request sampling state: the generator and the distinct tokens seen so far (kept as a growing
    array, so that a step's list of all requests' seen tokens is a concatenation, not a Python loop)."""

    def __init__(self, params: SamplingParams, prompt):
        self.params = params
        self.rng = SplitMix64(params.seed)
        self._set: set[int] = set()
        self._arr = np.empty(0, dtype=np.int32)
        self._n = 0
        if params.repetition_penalty != 1.0:
            first = list(dict.fromkeys(int(t) for t in prompt))
            self._set = set(first)
            self._arr = np.empty(max(64, 2 * len(first)), dtype=np.int32)
            self._arr[:len(first)] = first
            self._n = len(first)

    @property
    def seen(self) -> np.ndarray:
        return self._arr[:self._n]

    def note(self, token: int) -> None:
        if self.params.repetition_penalty != 1.0 and int(token) not in self._set:
            self._set.add(int(token))
            if self._n == len(self._arr):
                self._arr = np.concatenate([self._arr, np.empty(len(self._arr), dtype=np.int32)])
            self._arr[self._n] = int(token)
            self._n += 1


def sample_rows(ops, logits: torch.Tensor, samplers: list[RequestSampler]) -> list[int]:
    """One token per row of ``logits`` ([N, V], 32-bit, on the device).  Advances each
    non-greedy request's generator by one draw."""
    n = logits.shape[0]
    if n == 0:
        return []
    if all(s.params.plain_greedy for s in samplers):
        return ops.argmax(logits).tolist()
    dev = logits.device
    # one host buffer of 32-bit words for everything the kernel reads besides the logits, one copy:
    # [N x 4 params | N uniforms | N top_k | N + 1 offsets | seen tokens]
    offsets = [0]
    for s in samplers:
        offsets.append(offsets[-1] + len(s.seen))
    seen = np.concatenate([s.seen for s in samplers]) if offsets[-1] else np.zeros(1, dtype=np.int32)
    floats = []
    for s in samplers:
        floats += [s.params.temperature, s.params.top_p, s.params.min_p, s.params.repetition_penalty]
    floats += [0.0 if s.params.greedy else s.rng.next_f32() for s in samplers]
    ints = np.concatenate([np.asarray([s.params.top_k for s in samplers] + offsets, dtype=np.int32), seen])
    host = torch.empty(len(floats) + len(ints), dtype=torch.int32, pin_memory=(dev.type == "cuda"))
    host[:len(floats)].view(torch.float32).copy_(torch.tensor(floats, dtype=torch.float32))
    host[len(floats):].copy_(torch.from_numpy(ints))
    buf = host.to(dev, non_blocking=True)
    f = buf[:len(floats)].view(torch.float32)
    i0 = len(floats)
    params, u = f[:4 * n].view(n, 4), f[4 * n:5 * n]
    top_k = buf[i0:i0 + n]
    seen_offsets = buf[i0 + n:i0 + 2 * n + 1]
    seen_tokens = buf[i0 + 2 * n + 1:]
    out = ops.sample(logits, params, top_k, u, seen_offsets, seen_tokens)
    return out.tolist()
