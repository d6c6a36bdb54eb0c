from .api import KernelError, KernelSet, KernelTimeout, Routing

__all__ = ["KernelError", "KernelSet", "KernelTimeout", "Routing"]
