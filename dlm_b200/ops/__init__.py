"""Kernel backend.  ``native_ops()`` is the only backend the package has."""
from .native import KernelError, NativeOps


def native_ops(fast: bool = True) -> NativeOps:
    return NativeOps(fast=fast)


__all__ = ["KernelError", "NativeOps", "native_ops"]
