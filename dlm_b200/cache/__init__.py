from .manager import ModelCache

__all__ = ["ModelCache"]
