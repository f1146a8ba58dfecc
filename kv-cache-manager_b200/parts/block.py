"""Arrangement of parts in one layer.  ``PreNormBlock``: x += mixer(norm1(x)); x += ffn(norm2(x))
(``src/model/llama.cpp:104-124``).  The residual stream x is float32; a sub-layer's output is
not added at once but handed on as *pending* and added inside the next norm kernel."""
from __future__ import annotations

from typing import Optional

import torch

from .base import BLOCKS, Block, FeedForward, Mixer, Norm, SiteCache, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward) -> None:
        super().__init__()
        self.norm1 = self.add_child("norm1", norm1)
        self.mixer = self.add_child("mixer", mixer)
        self.norm2 = self.add_child("norm2", norm2)
        self.ffn = self.add_child("ffn", ffn)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                site: SiteCache) -> torch.Tensor:
        h = torch.empty(x.shape, dtype=ctx.dtype, device=x.device)
        self.norm1.forward(x, pending, h)
        y = self.mixer.forward(h, ctx, site)
        self.norm2.forward(x, y, h)
        return self.ffn.forward(h, ctx)
