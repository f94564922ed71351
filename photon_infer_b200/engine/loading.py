"""From a model folder to a model on the device with its cache and step function."""
from __future__ import annotations

from typing import List, Optional

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
    tensors = load_tensors(folder, model.declared(), model.dtype, dev, spec.ignored_tensors)
    model.load(tensors)
    return model


def random_model(config: dict, dtype: str = "bfloat16", device: str = "cuda:0", seed: int = 0,
                 init_std: float = 0.02, norm_std: float = 0.0) -> CausalLM:
    """A model of the configuration ``config`` (config.json form) with weights drawn on the device; no
    folder is written or read.  For measurements at large shapes; ``write_random_model`` is the
    random-weights mode that generation, replay and the tests use."""
    from ..config.registry import get_architecture
    from ..weights.random_init import random_tensors_on_device
    dev = require_cuda(device)
    arch = get_architecture((config.get("architectures") or [None])[0])
    cfg = arch.config_class.from_dict(config)
    model = CausalLM(arch.build_spec(cfg), _TORCH_DTYPES[dtype], dev)
    model.config = cfg
    ensure_built(model.kernel_modules())
    model.load(random_tensors_on_device(model.declared(), model.dtype, dev, seed, init_std, norm_std))
    return model


def pages_for(model: CausalLM, options: EngineOptions, max_model_len: int) -> List[int]:
    """Pages of each cache group: as given, or for ``max_cache_tokens``, or what the free memory holds.
    A group that keeps a window never holds more than the window and one step's tokens per request, so it
    gets no more pages than that; what it leaves of the memory goes to the groups that keep everything."""
    ps = options.block_size
    specs = CacheManager.group_specs(model.cache_needs(), [e.kv_from for e in model.spec.run])
    if not specs:
        return []

    def cap(spec) -> Optional[int]:
        if spec.window is None:
            return None
        per_request = -(-(spec.window + min(options.max_num_batched_tokens, max_model_len)) // ps) + 1
        return options.max_sequences * per_request

    def capped(n: int) -> List[int]:
        return [max(1, n if cap(s) is None else min(n, cap(s))) for s, _ in specs]

    if options.num_blocks is not None:
        return [options.num_blocks] * len(specs)
    if options.max_cache_tokens is not None:
        return capped((options.max_cache_tokens + ps - 1) // ps)
    es = torch.empty((), dtype=model.dtype).element_size()
    page_bytes = [len(entries) * 2 * s.n_kv_heads * s.head_dim * es * ps for s, entries in specs]
    free, _total = torch.cuda.mem_get_info(model.device)
    budget = int(free * options.gpu_memory_fraction)
    # no more than every live request at full length, and no more than 2^20 tokens unless asked for
    most = max(1, min(options.max_sequences * max_model_len, 1 << 20) // ps)
    pages = capped(min(most, budget // sum(page_bytes)))
    open_groups = [i for i, (s, _) in enumerate(specs) if cap(s) is None or pages[i] < cap(s)]
    if open_groups and len(open_groups) < len(specs):
        left = budget - sum(pages[i] * page_bytes[i] for i in range(len(specs)) if i not in open_groups)
        n = max(1, min(most, left // sum(page_bytes[i] for i in open_groups)))
        for i in open_groups:
            pages[i] = n if cap(specs[i][0]) is None else min(n, cap(specs[i][0]))
    return pages


def build_cache(model: CausalLM, options: EngineOptions, max_model_len: Optional[int] = None) -> CacheManager:
    mml = max_model_len or options.max_model_len or model.spec.max_position
    pages = pages_for(model, options, mml)
    return CacheManager(model.cache_needs(), [e.kv_from for e in model.spec.run], options.block_size,
                        pages if pages else 1, options.max_sequences, model.dtype, model.device)


def build_runner(folder: str, options: EngineOptions, model: Optional[CausalLM] = None) -> ModelRunner:
    """``model``: an already loaded model to build the cache and the step function around (``folder`` is
    then not read)."""
    options.validate()
    if model is None:
        model = load_model(folder, options.dtype, options.device)
    mml = options.max_model_len or model.spec.max_position
    return ModelRunner(model, build_cache(model, options, mml), mml, use_cuda_graphs=options.use_cuda_graphs)
