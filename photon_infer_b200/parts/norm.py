"""RMSNorm: ``y = w * (x / sqrt(mean(x^2) + eps))`` in 32-bit
(include/photon/ops/kernels/rmsnorm_kernel.hpp:71-86), fused with the residual sum
that precedes it (the reference runs a separate add kernel,
src/arch/transformer_block.cpp:270,295)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Norm, TensorSpec
from .registry import register_norm


class RMSNorm(Norm):
    kernel_modules = ("elementwise",)

    def __init__(self, size: int, eps: float, weight_name: str = "weight"):
        self.size = size
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.size,), role="vector", init="norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return self.add_forward(None, x, out_dtype)

    def add_forward(self, delta, residual, out_dtype):
        out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        ops.add_rmsnorm(delta, residual, self.weight, self.eps, out)
        return out

    def add_forward_rows(self, delta, residual, rows, out_dtype):
        out = torch.empty((rows.numel(), residual.shape[1]), dtype=out_dtype, device=residual.device)
        ops.add_rmsnorm(delta, residual, self.weight, self.eps, out, rows=rows)
        return out


register_norm("rms_norm", RMSNorm)
