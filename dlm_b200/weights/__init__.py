from .loader import load_model, random_model
from .random_init import random_tensor, write_random_model
from .safetensors_io import SafetensorsError, TensorStore, save_file

__all__ = ["load_model", "random_model", "random_tensor", "write_random_model", "SafetensorsError", "TensorStore",
           "save_file"]
