"""Sampling of the next token from 32-bit logits, on the device.

Greedy takes the first maximum (src/arch/llama_model.cpp:304-328; src/ops/kernels/cuda/
sampling_kernel.cu:36-138).  Temperature sampling follows the reference's command line
(demo/llama_infer.cpp:78-101): ``p_i = exp((l_i - max) / T) / sum`` and the first index
whose running sum reaches a uniform number.  There the number comes from ``rand()``
seeded by the clock; here it comes from a counter-based generator keyed by (seed,
request, index of the generated token), so a request's tokens can be reproduced and do
not depend on what else is in the batch.  The reference parses ``top_p`` and ignores it
(web/web_server.cpp:447-448); it is not offered here.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, request_id: int, index: int) -> float:
    """A number in [0, 1) that depends only on its three keys; 24 bits, exact in float32."""
    h = _splitmix64(seed & _MASK)
    h = _splitmix64(h ^ (request_id & _MASK))
    h = _splitmix64(h ^ (index & _MASK))
    return (h >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], uniforms: Sequence[float]) -> torch.Tensor:
        """``logits`` float32 [rows, vocab] on the device; returns int32 [rows] on the device."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if rows == 0:
            return out
        if all(t <= 0 for t in temperatures):
            ops.sample(logits, None, None, out)
            return out
        host = torch.tensor([list(temperatures), list(uniforms)], dtype=torch.float32).pin_memory()
        dev = host.to(self.device, non_blocking=True)
        ops.sample(logits, dev[0], dev[1], out)
        return out
