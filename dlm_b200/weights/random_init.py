"""Seeded random weights.

Every element is a pure function of ``(seed, tensor name, flat index)``: a
SplitMix64-style mix of a per-tensor key and the index gives two uniforms, a
Box-Muller transform in double precision gives a normal deviate.  Linear
weights and biases are N(0, 0.02), norm weights 1 + N(0, 0.02).  The same
function runs on the host (to write a model folder) and on the device (to fill a
large model in place without a file), so both see the same weights up to the
last bit of the platform's double-precision ``log``/``cos``.

The reference's own synthetic model draws uniform(-0.02, 0.02) from a single
SplitMix64 stream in tensor order (src/main.rs:220-239, 433-449); a stream
cannot be filled in parallel or by name, hence the counter-based form here.
"""
from __future__ import annotations

import hashlib
import json
import math
import os

import torch

from .safetensors_io import save_file

_GOLDEN = 0x9E3779B97F4A7C15
_C1 = 0xBF58476D1CE4E5B9
_C2 = 0x94D049BB133111EB
_CHUNK = 1 << 24


def _s64(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(z: torch.Tensor, n: int) -> torch.Tensor:
    return (z >> n) & ((1 << (64 - n)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _s64(_C1)
    z = (z ^ _lsr(z, 27)) * _s64(_C2)
    return z ^ _lsr(z, 31)


def tensor_key(seed: int, name: str) -> int:
    h = int.from_bytes(hashlib.blake2b(name.encode("utf-8"), digest_size=8).digest(), "little")
    return _s64(h ^ ((seed * _GOLDEN) & ((1 << 64) - 1)))


def random_tensor(name: str, shape, init: str, seed: int, device="cpu", dtype=torch.float32,
                  std: float = 0.02) -> torch.Tensor:
    numel = 1
    for s in shape:
        numel *= int(s)
    out = torch.empty(numel, dtype=dtype, device=device)
    key = tensor_key(seed, name)
    mean = 1.0 if init == "norm" else 0.0
    for start in range(0, numel, _CHUNK):
        n = min(_CHUNK, numel - start)
        i = torch.arange(start, start + n, dtype=torch.int64, device=device)
        a = _mix((2 * i + 1) * _s64(_GOLDEN) + key)
        b = _mix((2 * i + 2) * _s64(_GOLDEN) + key)
        u1 = (_lsr(a, 40).to(torch.float64) + 0.5) / float(1 << 24)
        u2 = (_lsr(b, 40).to(torch.float64) + 0.5) / float(1 << 24)
        z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
        out[start:start + n] = (mean + std * z).to(dtype)
    return out.reshape(tuple(int(s) for s in shape))


def random_state_dict(param_specs: dict, seed: int, dtype=torch.float32, device="cpu",
                      include_optional: bool = True, skip=()) -> dict[str, torch.Tensor]:
    out = {}
    for name, p in param_specs.items():
        if name in skip or (p.optional and not include_optional):
            continue
        out[name] = random_tensor(name, p.shape, p.init, seed, device=device, dtype=dtype)
    return out


def write_random_model(config, seed: int, out_dir: str, dtype=torch.float32) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for a typed config and a seed.
    A tied model gets no ``lm_head.weight``; optional biases are written."""
    from ..parts.base import Runtime
    from ..parts.model import DecoderModel
    from ..registry import spec_of_config
    spec = spec_of_config(config)
    model = DecoderModel(spec, Runtime("cpu", torch.float32, ops=None))
    skip = (spec.lm_head_name,) if spec.tie_word_embeddings else ()
    tensors = random_state_dict(model.param_specs(), seed, dtype=dtype, skip=skip)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), {"format": "pt", "seed": str(seed)})
    return out_dir
