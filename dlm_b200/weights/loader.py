"""Weights by tensor name: from a model folder, or drawn from a seed in place."""
from __future__ import annotations

import torch

from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..registry import resolve, spec_of_config
from .random_init import random_tensor
from .safetensors_io import TensorStore


def load_model(path: str, rt: Runtime):
    """(config, model) for a folder with ``config.json`` and ``*.safetensors``.  The model
    class is whatever the registry maps the config's architecture to.  Tensors are read by
    name; matrices are kept in the runtime's dtype, norm weights and biases in 32-bit.  A
    checkpoint that does not fit raises one ``WeightError`` listing every fault."""
    _, cfg, spec = resolve(path)
    model = DecoderModel(spec, rt)
    store = TensorStore(path)
    try:
        model.check({n: store.info(n) for n in store.names()})
        model.load(store.tensor, store.names())
    finally:
        store.close()
    return cfg, model


def random_model(config, seed: int, rt: Runtime):
    """(config, model) with every tensor drawn on the runtime's device from ``seed`` (the same
    values ``write_random_model`` would put in a folder)."""
    spec = spec_of_config(config)
    model = DecoderModel(spec, rt)
    specs = model.param_specs()
    names = [n for n, p in specs.items() if not (n == spec.lm_head_name and spec.tie_word_embeddings)]
    store_dtype = rt.dtype

    def get(name):
        p = specs[name]
        return random_tensor(name, p.shape, p.init, seed, device=rt.device,
                             dtype=store_dtype if p.init == "linear" else torch.float32)

    model.load(get, names)
    return config, model
