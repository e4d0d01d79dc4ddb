from .engine import Engine, generate, make_runtime

__all__ = ["Engine", "generate", "make_runtime"]
