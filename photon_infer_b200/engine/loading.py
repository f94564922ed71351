"""From a model folder to a model on the device with its cache and step function."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.manager import CacheManager
from ..config.engine_options import EngineOptions
from ..config.registry import load_config
from ..csrc.build import ensure_built
from ..errors import ErrorCode, PhotonError
from ..models.model import CausalLM
from ..weights.loader import load_tensors
from .runner import ModelRunner

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def require_cuda(device: str) -> torch.device:
    if not torch.cuda.is_available():
        raise PhotonError(ErrorCode.CUDA_ERROR, "no CUDA device is visible; this engine has no CPU path")
    dev = torch.device(device)
    if dev.type != "cuda":
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"device must be a CUDA device, got {device!r}")
    torch.cuda.set_device(dev)
    return dev


def load_model(folder: str, dtype: str = "bfloat16", device: str = "cuda:0") -> CausalLM:
    """Reads ``config.json``, picks the model by ``architectures[0]``, compiles the kernels it
    needs (first call only) and loads ``model.safetensors`` by tensor name."""
    dev = require_cuda(device)
    arch, config = load_config(folder)
    spec = arch.build_spec(config)
    model = CausalLM(spec, _TORCH_DTYPES[dtype], dev)
    model.config = config
    ensure_built(model.kernel_modules())
    tensors = load_tensors(folder, model.declared(), model.dtype, dev)
    model.load(tensors)
    return model


def pages_for(model: CausalLM, options: EngineOptions, max_model_len: int) -> int:
    """Pages per group: as given, or for ``max_cache_tokens``, or what the free memory holds."""
    ps = options.block_size
    if options.num_blocks is not None:
        return options.num_blocks
    if options.max_cache_tokens is not None:
        return (options.max_cache_tokens + ps - 1) // ps
    needs = model.cache_needs()
    es = torch.empty((), dtype=model.dtype).element_size()
    per_token = sum(2 * p.n_kv_heads * p.head_dim * es for p, _ in needs if p is not None)
    if per_token == 0:
        return 1
    free, _total = torch.cuda.mem_get_info(model.device)
    budget = int(free * options.gpu_memory_fraction)
    # no more than every live request at full length, and no more than 2^20 tokens unless asked for
    tokens = min(budget // per_token, options.max_sequences * max_model_len, 1 << 20)
    return max(1, tokens // ps)


def build_cache(model: CausalLM, options: EngineOptions, max_model_len: Optional[int] = None) -> CacheManager:
    mml = max_model_len or options.max_model_len or model.spec.max_position
    return CacheManager(model.cache_needs(), [e.kv_from for e in model.spec.run], options.block_size,
                        pages_for(model, options, mml), options.max_sequences, model.dtype, model.device)


def build_runner(folder: str, options: EngineOptions) -> ModelRunner:
    options.validate()
    model = load_model(folder, options.dtype, options.device)
    mml = options.max_model_len or model.spec.max_position
    return ModelRunner(model, build_cache(model, options, mml), mml, use_cuda_graphs=options.use_cuda_graphs)
