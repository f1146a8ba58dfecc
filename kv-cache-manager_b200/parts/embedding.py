"""Token embedding (gather into the float32 residual stream, no scaling:
``src/cuda/kernels.cu:27-32``) and the output head (logits in float32 for the wanted rows only:
``src/model/llama.cpp:126-128``)."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import Part, StepContext
from .linear import matmul_nt


class Embedding(Part):
    def __init__(self, vocab: int, hidden: int) -> None:
        super().__init__()
        self.vocab, self.hidden = vocab, hidden
        self.declare("weight", (vocab, hidden), ("normal", 0.02), "table")

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.rows, self.hidden), dtype=torch.float32, device=ctx.tokens.device)
        K.embed(ctx.tokens, self.param("weight"), x)
        return x


class LMHead(Part):
    """logits = h W^T in float32.  ``weight`` may alias the embedding table (tied)."""

    def __init__(self, hidden: int, vocab: int) -> None:
        super().__init__()
        self.vocab, self.hidden = vocab, hidden
        self.declare("weight", (vocab, hidden), ("normal", 0.02), "matrix")

    def forward(self, h: torch.Tensor, ctx: Optional[StepContext] = None) -> torch.Tensor:
        return matmul_nt(h, self.param("weight"), torch.float32, ctx.options if ctx else {})
