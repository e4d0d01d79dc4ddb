"""dlm_b200: a single-GPU inference engine for Qwen2-MoE on NVIDIA B200 (sm_100a)."""
from .config import ConfigError, Qwen2MoeConfig
from .registry import architectures, register_architecture, register_part, resolve

__version__ = "0.1.0"


def __getattr__(name):
    # heavy pieces are imported on first use
    if name in ("Engine", "generate", "make_runtime"):
        from . import engine
        return getattr(engine, name)
    if name in ("SamplingParams",):
        from . import sampling
        return getattr(sampling, name)
    raise AttributeError(name)


__all__ = ["ConfigError", "Qwen2MoeConfig", "Engine", "generate", "SamplingParams", "architectures",
           "register_architecture", "register_part", "resolve"]
