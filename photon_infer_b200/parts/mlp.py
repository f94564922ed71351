"""Dense SwiGLU feed-forward: ``down(silu(gate(h)) * up(h))``
(src/arch/transformer_block.cpp:282-291; include/photon/ops/kernels/swiglu_kernel.hpp:
67-76).  Gate and up are one fused matrix on the device, so ``h`` is read once."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward, StepContext, TensorSpec
from .linear import project
from .registry import register_feed_forward


class SwiGLUFeedForward(FeedForward):
    kernel_modules = ("elementwise",)

    def required_kernels(self, dtype):
        return ["elementwise"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return [TensorSpec("gate_proj.weight", (I, H)), TensorSpec("up_proj.weight", (I, H)),
                TensorSpec("down_proj.weight", (H, I))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ops.linear_swiglu(h, self.w_gate_up)
        return project(act, self.w_down)


register_feed_forward("swiglu", SwiGLUFeedForward)
