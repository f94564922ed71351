from .loader import load_tensors
from .random_init import write_random_model
from .safetensors_io import SafetensorsFile, open_model_files, write_safetensors

__all__ = ["load_tensors", "write_random_model", "SafetensorsFile", "open_model_files", "write_safetensors"]
