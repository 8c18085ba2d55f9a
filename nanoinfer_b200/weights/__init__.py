from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, save_safetensors
from .loader import WeightError, load_tensors
from .random_init import random_tensors, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "open_model_files", "save_safetensors",
           "WeightError", "load_tensors", "random_tensors", "write_random_model"]
