"""Weight matrices of the projections, ``y = x W^T`` with ``W [out, in]`` and no bias
(include/photon/ops/matmul.hpp:64-109)."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


def project(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    return ops.linear(x, weight, out=out, out_dtype=out_dtype)
