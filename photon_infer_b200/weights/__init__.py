from .loader import load_tensors
from .random_init import random_tensors_on_device, write_random_model
from .safetensors_io import SafetensorsFile, open_model_files, write_safetensors

__all__ = ["load_tensors", "write_random_model", "random_tensors_on_device", "SafetensorsFile", "open_model_files",
           "write_safetensors"]
