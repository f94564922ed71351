"""Random-weights mode: writes a model folder (``config.json``, ``model.safetensors``)
from a configuration and a seed.

The reference draws N(0, 0.02) for every tensor, norms included, in its tests only
(tests/model/test_llama_model.cpp:31-42).  Here each tensor has its own generator,
seeded from (seed, tensor name), so the values of one tensor do not depend on which
other tensors the model has; matrices are N(0, init_std), norm weights are ones or
``1 + N(0, norm_std)``.  Values are rounded to the storage dtype (bfloat16 by
default) before writing, so a float32 run and a bfloat16 run read the same numbers.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import torch

from ..config.registry import get_architecture
from ..errors import ErrorCode, PhotonError
from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensor(spec: TensorSpec, name: str, seed: int, init_std: float, norm_std: float,
                  dtype: torch.dtype) -> torch.Tensor:
    g = _generator(seed, name)
    if spec.role == "int":
        return torch.zeros(spec.shape, dtype=torch.int32)
    if spec.init == "zeros":
        t = torch.zeros(spec.shape, dtype=torch.float32)
    elif spec.init == "norm":
        t = torch.ones(spec.shape, dtype=torch.float32)
        if norm_std > 0:
            t += norm_std * torch.randn(spec.shape, generator=g, dtype=torch.float32)
    elif spec.init == "normal":
        t = init_std * torch.randn(spec.shape, generator=g, dtype=torch.float32)
    else:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"tensor {name}: unknown init {spec.init!r}")
    return t.to(dtype)


def write_random_model(folder: str, config, seed: int = 0, init_std: float = 0.02, norm_std: float = 0.0,
                       dtype: str = "bfloat16", architecture: Optional[str] = None) -> Dict[str, tuple]:
    """``config`` is a typed configuration (e.g. ``LlamaConfig``) or a dict in config.json form."""
    from ..models.model import declared_tensors
    if isinstance(config, dict):
        name = architecture or (config.get("architectures") or [None])[0]
        arch = get_architecture(name)
        config = arch.config_class.from_dict(config)
    else:
        arch = get_architecture(architecture or config.architecture)
    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(dtype)
    if store is None:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"storage dtype must be bfloat16 or float32, got {dtype!r}")
    spec = arch.build_spec(config)
    declared = declared_tensors(spec)
    tensors = {name: random_tensor(ts, name, seed, init_std, norm_std, store) for name, ts in declared.items()}
    os.makedirs(folder, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed, "init_std": init_std, "norm_std": norm_std})
    return {n: tuple(t.shape) for n, t in tensors.items()}


def random_tensors_on_device(declared: Dict[str, TensorSpec], run_dtype: torch.dtype, device, seed: int = 0,
                             init_std: float = 0.02, norm_std: float = 0.0) -> Dict[str, torch.Tensor]:
    """The tensors a model declares, drawn on the device itself: for measurements at sizes whose weight file
    would take longer to write and read than the run (a Llama 3.1 8B shape is 16 GB).  Same distributions as
    ``write_random_model`` and the same storage rule as the loader, but the device's generator: the values
    differ from those of a folder written with the same seed."""
    dev = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for i, (name, spec) in enumerate(declared.items()):
        g = torch.Generator(device=dev)
        digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
        g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
        if spec.role == "int":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=dev)
            continue
        dtype = torch.float32 if (run_dtype == torch.float32 or spec.role == "vector") else run_dtype
        if spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=dtype, device=dev)
        elif spec.init == "norm":
            t = torch.ones(spec.shape, dtype=dtype, device=dev)
            if norm_std > 0:
                t += norm_std * torch.randn(spec.shape, generator=g, dtype=dtype, device=dev)
        elif spec.init == "normal":
            t = torch.empty(spec.shape, dtype=dtype, device=dev).normal_(0.0, init_std, generator=g)
        else:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"tensor {name}: unknown init {spec.init!r}")
        out[name] = t
    return out
