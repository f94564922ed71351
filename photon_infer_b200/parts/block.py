"""Pre-norm arrangement of a layer: ``x += mixer(norm1(x)); x += ff(norm2(x))``
(src/arch/transformer_block.cpp:199-296).  Each residual sum is handed to the norm
that follows it, which does both in one pass over the row, in 32-bit."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import Block, FeedForward, LayerCache, Mixer, Norm, Part, StepContext
from .registry import register_block


class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward):
        self.norm1, self._mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self) -> Dict[str, Part]:
        return {"norm1": self.norm1, "mixer": self._mixer, "norm2": self.norm2, "feed_forward": self.feed_forward}

    def mixer(self) -> Mixer:
        return self._mixer

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        # a part may take the residual sum and the norm into its first kernel (decode steps)
        if self._mixer.fuses_norm(self.norm1, residual, ctx, cache):
            a, residual = self._mixer.forward_with_norm(residual, delta, self.norm1, ctx, cache)
        else:
            h = self.norm1.add_forward(delta, residual, ctx.dtype)
            a = self._mixer.forward(h, ctx, cache)
        if self.feed_forward.fuses_norm(self.norm2, residual, ctx):
            d, residual = self.feed_forward.forward_with_norm(residual, a, self.norm2, ctx)
        else:
            h2 = self.norm2.add_forward(a, residual, ctx.dtype)
            d = self.feed_forward.forward(h2, ctx)
        return residual, d


register_block("pre_norm", PreNormBlock)
