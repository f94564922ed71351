"""Rotary position encoding.

The reference rotates neighbouring pairs with a fixed base of 10000 and a table of
sines and cosines per layer (include/photon/ops/kernels/rope_kernel.hpp:54-84,
143-165).  Here the base, the frequency scaling and the pairing are parameters, one
table of inverse frequencies is shared by all layers, and the angle ``pos *
inv_freq[j]`` with its sine and cosine is computed in 32-bit inside the kernel.

``inverse_frequencies`` follows the published Llama 3.1 rule for ``rope_type ==
"llama3"``: with wavelength ``lam = 2*pi / f`` and ``orig`` the original maximum
position, ``lam > orig / low_freq_factor`` gives ``f / factor``, ``lam < orig /
high_freq_factor`` keeps ``f``, and between them ``s = (orig / lam - low) / (high -
low)``, ``f' = (1 - s) * f / factor + s * f``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import PositionEncoding
from .registry import register_position_encoding


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """float64 arithmetic on the host, returned as float32 ``[head_dim / 2]``."""
    out = []
    for j in range(head_dim // 2):
        f = float(theta) ** (-2.0 * j / head_dim)
        if scaling is not None:
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            lam = 2.0 * math.pi / f
            if lam > orig / low:
                f = f / factor
            elif lam >= orig / high:
                s = (orig / lam - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


class RotaryEncoding(PositionEncoding):
    kernel_modules = ("rope_kv",)

    def __init__(self, head_dim: int, theta: float, scaling: Optional[dict] = None, interleaved: bool = False):
        if head_dim % 2:
            raise ValueError("rotary encoding needs an even head_dim")
        self.head_dim = head_dim
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.interleaved = bool(interleaved)
        self.inv_freq_host = inverse_frequencies(head_dim, self.theta, self.scaling)
        self.inv_freq: Optional[torch.Tensor] = None
        self._table: Optional[torch.Tensor] = None

    def to_device(self, device) -> None:
        self.inv_freq = self.inv_freq_host.to(device)
        self._table = None

    def table(self, positions: int) -> torch.Tensor:
        """``(cos, sin)`` for positions below a power of two that covers ``positions`` (grown on demand,
        built on the device with the kernels' own expression): for kernels that look angles up."""
        if getattr(self, "_table", None) is None or self._table.shape[0] < positions:
            count = 1024
            while count < positions:
                count *= 2
            self._table = ops.rope_table(self.inv_freq, count)
        return self._table

    def apply(self, q, k, positions) -> None:
        """In place; ``q [T, n_q, d]`` and ``k [T, n_kv, d]`` may be views with any row stride."""
        n_q = q.shape[1] if q is not None else 0
        n_kv = k.shape[1] if k is not None else 0
        ops.rope_kv_write(q, k, None, positions, self.inv_freq, self.interleaved, None, None, None,
                          n_q, n_kv, self.head_dim, None)


register_position_encoding("rotary", RotaryEncoding)
