from .safetensors_io import SafetensorsError, SafetensorsFile, open_checkpoint, save_file
from .loader import WeightError, load_bound_tensors, storage_dtype
from .random_init import random_tensor, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "open_checkpoint", "save_file", "WeightError",
           "load_bound_tensors", "storage_dtype", "random_tensor", "write_random_model"]
