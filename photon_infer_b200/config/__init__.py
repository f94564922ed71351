from .engine_options import EngineOptions, normalize_dtype
from .model_config import LlamaConfig, RopeScaling, read_config_json
from .registry import (Architecture, get_architecture, load_config, register_architecture,
                       registered_architectures)

__all__ = ["EngineOptions", "normalize_dtype", "LlamaConfig", "RopeScaling", "read_config_json",
           "Architecture", "get_architecture", "load_config", "register_architecture",
           "registered_architectures"]
