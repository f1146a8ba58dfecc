"""RMSNorm with the residual add that precedes it fused in.

out = w * round(x * rsqrt(mean(x^2) + eps)); statistics in float32 over the float32 residual
stream (the reference's kernel, ``src/cuda/kernels.cu:34-49``; its separate residual kernel,
``:84-88``, is folded into this one).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import NORMS, Norm


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, hidden: int, eps: float, init=("ones",)) -> None:
        super().__init__()
        self.hidden, self.eps = hidden, float(eps)
        self.declare("weight", (hidden,), init, "vector")

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        K.rmsnorm(x, pending, self.param("weight"), out, self.eps, rows)
