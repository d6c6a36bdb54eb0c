from .api import KernelError, KernelSet, Routing

__all__ = ["KernelError", "KernelSet", "Routing"]
