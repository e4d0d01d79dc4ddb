"""The plain implementation against outputs of the reference's own CUDA model code.

tests/golden/tiny_*_reference_kernels.npz hold, for each tiny configuration with its window
switched off, the residual stream after the last layer as vedantnimbarte/dlm's src/gpu/kernels.cu
computed it on a B200, token by token with its own key/value history (made once by
tests/golden/make_golden.py, which says what the files pin and what they cannot).  The files
depend on the seeded weights; a digest of the tensors guards against a silent change of the
generator.
"""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen2_moe as plain
from tiny_configs import TINY

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _digest(tensors) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].contiguous().numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("name", list(TINY))
def test_plain_matches_reference_kernels(name, tiny_folders):
    path = os.path.join(GOLDEN, f"tiny_{name}_reference_kernels.npz")
    gold = np.load(path)
    raw, tensors = plain.load_folder(tiny_folders[name])
    assert _digest(tensors) == str(gold["weights_sha256"]), "the seeded weights changed: make the golden files again"
    raw = dict(raw, use_sliding_window=False)
    tokens = gold["tokens"].tolist()
    want = torch.from_numpy(gold["hidden"]).to(torch.float64)
    model = plain.PlainModel((raw, tensors), compute=torch.float64)
    got = model.hidden_states(tokens)
    margins = model.router_margins(tokens)
    # the reference computes in 32-bit: a routing choice within 1e-6 of a tie may fall the other way
    keep = margins >= 1e-6
    assert int(keep.sum()) >= len(tokens) - 1
    scale = float(want.abs().max())
    diff = float((got[keep] - want[keep]).abs().max())
    assert diff <= 2e-6 * max(scale, 1.0), f"tiny {name}: max abs diff {diff:.3e} (values up to {scale:.3f})"
    # and the two differ where they should: with a window shorter than the prompt the model is another function
    if TINY[name]["cfg"].get("use_sliding_window") and TINY[name]["cfg"]["sliding_window"] < len(tokens):
        windowed = plain.PlainModel((dict(raw, use_sliding_window=True), tensors), compute=torch.float64)
        assert float((windowed.hidden_states(tokens) - want).abs().max()) > 1e-4
