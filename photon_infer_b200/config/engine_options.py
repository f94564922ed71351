"""Options of the engine (not of the model).

Names follow the reference where it has them: ``max_batch_size``, ``chunk_size``
(default 256) and ``max_sequences`` (default 32) are the constructor arguments of
``ContinuousBatchEngine`` / ``ContinuousBatchScheduler``
(include/photon/scheduler/continuous_batch_engine.hpp:57-66,
include/photon/scheduler/continuous_batch_scheduler.hpp:80-100); ``num_blocks`` and
``block_size`` are the arguments of ``LLaMAModel::init_paged_cache``
(src/arch/llama_model.cpp:453).  ``max_num_batched_tokens`` (a token budget per
step) and ``max_model_len`` have no counterpart there.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

from ..errors import ErrorCode, PhotonError


@dataclasses.dataclass
class EngineOptions:
    dtype: str = "bfloat16"                 # "bfloat16" | "float32"
    block_size: int = 16                    # tokens per cache page
    num_blocks: Optional[int] = None        # pages per cache group; None: from max_cache_tokens or memory
    max_cache_tokens: Optional[int] = None  # alternative to num_blocks: tokens the pool must hold
    gpu_memory_fraction: float = 0.85       # used when neither of the two above is given
    max_sequences: int = 32                 # live requests (rows of the block table, state slots)
    max_batch_size: int = 32                # requests in one step
    chunk_size: int = 256                   # longest prompt portion of one request in one step
    max_num_batched_tokens: int = 2048      # token budget of one step over all requests
    max_model_len: Optional[int] = None     # longest request; None: max_position_embeddings
    seed: int = 0
    use_cuda_graphs: bool = True
    async_decode: bool = True               # enqueue the next decode step before reading the last one's ids
    device: str = "cuda:0"

    def validate(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        for name in ("block_size", "max_sequences", "max_batch_size", "chunk_size", "max_num_batched_tokens"):
            if getattr(self, name) <= 0:
                raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"{name} must be positive")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "num_blocks must be positive")


def normalize_dtype(name: str) -> str:
    table = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32", "f32": "float32"}
    if name not in table:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"unknown dtype {name!r} (bfloat16 or float32)")
    return table[name]
