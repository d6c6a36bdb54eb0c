from .safetensors_io import SafetensorsError, SafetensorsFile, open_checkpoint, save_file
from .loader import (WeightError, apply_binding, bind_tensors, load_bound_tensors, register_weight_transform,
                     storage_dtype, weight_transforms)
from .random_init import random_checkpoint_tensors, random_tensor, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "open_checkpoint", "save_file", "WeightError",
           "apply_binding", "bind_tensors", "load_bound_tensors", "register_weight_transform", "storage_dtype",
           "weight_transforms", "random_checkpoint_tensors", "random_tensor", "write_random_model"]
