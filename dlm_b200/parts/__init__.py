"""Built-in parts.  Importing this package registers them."""
from . import attention, block, ffn, norm, rope  # noqa: F401
from .base import (CacheTensor, FeedForward, GroupView, Mixer, Norm, PagedCache, PagedKV, PagedView, ParamSpec, Part, PartSpec,
                   PositionEncoding, RequestState, Runtime, StepBatch, StepContext)
from .model import DecoderModel, LayerCall, ModelSpec, WeightError

__all__ = ["CacheTensor", "PagedCache", "FeedForward", "GroupView", "Mixer", "Norm", "PagedKV", "PagedView", "ParamSpec", "Part", "PartSpec",
           "PositionEncoding", "RequestState", "Runtime", "StepBatch", "StepContext", "DecoderModel", "LayerCall",
           "ModelSpec", "WeightError"]
