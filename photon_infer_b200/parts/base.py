"""Interfaces of the parts a layer is put together from.

A layer is a *block* that arranges a *mixer* (attention here), a *feed-forward* and
*norms*; a mixer may use a *position encoding*.  Every part gets its sizes and
constants as constructor parameters, declares the weight tensors it needs
(``tensor_specs``) and receives them by local name (``load``).  No part knows which
model it is in: the weight-name prefix, the layer index and the cache it reads are
handed to it from outside.

The reference builds each block from fixed operator members
(include/photon/arch/transformer_block.hpp:53-218); the split into exchangeable
parts has no counterpart there.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ----------------------------------------------------------------------------- weights

@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """One weight tensor of a part.

    ``role``: ``"matrix"`` tensors are operands of matrix products or lookup tables
    and are held in the run dtype; ``"vector"`` tensors (norm weights) keep 32-bit
    storage when the file has it; ``"int"`` tensors are integer tables, held as int32.
    ``init`` tells the random-weights mode how to fill it: ``"normal"`` (N(0, std)),
    ``"norm"`` (ones, or 1 + N(0, norm_std)), ``"zeros"``.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


# ----------------------------------------------------------------------------- caches

@dataclasses.dataclass(frozen=True)
class PagedCacheSpec:
    """What a mixer needs of the paged cache, per token: keys and values of
    ``n_kv_heads * head_dim`` each.  ``window`` None: every earlier key stays
    visible; an integer: only the last ``window`` keys do, and pages behind the
    window are given back.  Layers with equal specs share one group of pages."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """Fixed-size state of one request in one layer (shape without the slot axis)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclasses.dataclass
class GroupView:
    """Device-side view of one cache group for the current step."""
    block_table: torch.Tensor       # int32 [S, max_pages]; -1 where no page is held
    slot_mapping: torch.Tensor      # int32 [T]; page * page_size + offset of each token of the step
    page_size: int
    num_pages: int
    max_pages_per_seq: int


@dataclasses.dataclass
class LayerCache:
    """What one entry of the run list gets for its mixer."""
    group: Optional[int] = None             # index into StepContext.groups
    k: Optional[torch.Tensor] = None        # [num_pages, n_kv, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    shared: bool = False                    # true: another entry wrote these pages; do not write
    state: Optional[torch.Tensor] = None    # [max_sequences, *StateSpec.shape]


@dataclasses.dataclass
class StepContext:
    """Everything a part may read about the current step.

    Token-major arrays have one entry per token of the step (``T``); sequence-major
    arrays one per request in the step (``S``), in batch order.
    """
    num_tokens: int
    num_seqs: int
    dtype: torch.dtype                      # run dtype of activations and caches
    token_ids: torch.Tensor                 # int32 [T]
    positions: torch.Tensor                 # int32 [T] position of each token in its request
    token_seq: torch.Tensor                 # int32 [T] index of the token's request in the batch
    cu_tokens: torch.Tensor                 # int32 [S+1] first token of each request in the step
    context_lens: torch.Tensor              # int32 [S] tokens of the request after this step
    state_slots: torch.Tensor               # int32 [S] slot of the request's fixed-size state
    groups: List[GroupView]
    # host copies, for choosing kernels and grids
    host_query_lens: Sequence[int] = ()
    host_context_lens: Sequence[int] = ()
    host_start_positions: Sequence[int] = ()
    max_query_len: int = 0
    max_context_len: int = 0
    error_flag: Optional[torch.Tensor] = None   # int32 [4] written by kernels on bad indices
    scratch: Optional[object] = None            # engine.workspace.Workspace


# ----------------------------------------------------------------------------- parts

class Part:
    """Base of all parts: declared tensors in, device tensors held."""

    #: names of the CUDA modules (files under csrc/) the part launches
    kernel_modules: Tuple[str, ...] = ()

    def required_kernels(self, dtype: torch.dtype) -> List[object]:
        """Modules to compile before the first step: names, or (name, definitions) pairs."""
        return list(self.kernel_modules)

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors of ``tensor_specs`` by local name, on the device."""

    def weight_bytes(self) -> int:
        """Bytes a step reads of this part's weights (for the roofline)."""
        return 0


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """``x`` is the 32-bit residual stream ``[T, H]``; returns the normed rows."""
        raise NotImplementedError

    def add_forward(self, delta: Optional[torch.Tensor], residual: torch.Tensor,
                    out_dtype: torch.dtype) -> torch.Tensor:
        """``residual += delta`` (in 32-bit, in place), then ``forward(residual)``."""
        if delta is not None:
            residual.add_(delta.to(residual.dtype))
        return self.forward(residual, out_dtype)

    def add_forward_rows(self, delta: Optional[torch.Tensor], residual: torch.Tensor,
                         rows: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """Same as ``add_forward`` for the listed rows only; returns ``[len(rows), H]``."""
        r = residual.index_select(0, rows.long())
        d = delta.index_select(0, rows.long()) if delta is not None else None
        return self.add_forward(d, r, out_dtype)


class PositionEncoding(Part):
    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        """Encode in place: ``q [T, n_q, d]``, ``k [T, n_kv, d]`` (views with a row stride)."""
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """``h [T, H]`` normed input in the run dtype; returns ``[T, H]`` to add to the residual."""
        raise NotImplementedError

    # Optional fast path.  A mixer that can take the residual sum and the norm into its first kernel
    # answers True and implements forward_with_norm; the block then skips the separate norm pass.
    def fuses_norm(self, norm: Norm, residual: torch.Tensor, ctx: StepContext, cache: LayerCache) -> bool:
        return False

    def forward_with_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], norm: Norm,
                          ctx: StepContext, cache: LayerCache) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(output, new residual)`` where the new residual is ``residual + delta``."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def fuses_norm(self, norm: Norm, residual: torch.Tensor, ctx: StepContext) -> bool:
        return False

    def forward_with_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], norm: Norm,
                          ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError


class Block(Part):
    """Arrangement of parts in a layer.  ``forward`` gets the 32-bit residual stream
    and the not-yet-added output of the previous block, and returns the same pair, so
    that every residual sum is fused with the norm that follows it."""

    def parts(self) -> Dict[str, Part]:
        raise NotImplementedError

    def mixer(self) -> Mixer:
        raise NotImplementedError

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError
