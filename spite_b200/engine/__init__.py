from .batch import Segment, StepBatch, build_step_batch
from .executor import ContextOverflow, Engine, StepEntry, StepError
from ..kernels.api import KernelTimeout
from .model import Model, resolve_dtype

__all__ = ["Segment", "StepBatch", "build_step_batch", "ContextOverflow", "Engine", "StepEntry",
           "StepError", "KernelTimeout", "Model", "resolve_dtype"]
