"""Position encodings a mixer can be given.

``RotaryEmbedding``: angle(pos, j) = pos * inv_freq[j], inv_freq[j] = theta^(-2j / rotary_dim),
applied to pairs (j, j + rotary_dim/2) ("half", the reference's pairing,
``src/cuda/kernels.cu:51-70``) or (2j, 2j+1) ("interleaved") of the first ``rotary_dim``
elements of every q and k head.  The frequency table is float32, computed once on the host in
float64; a scaled variant only needs another table.  ``NoPositionEncoding`` leaves q and k as
they are.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


@POSITION_ENCODINGS.register("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None,
                 pairing: str = "half") -> None:
        super().__init__()
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing '{pairing}'")
        self.interleaved = pairing == "interleaved"
        self.inv_freq: Optional[torch.Tensor] = None

    def frequency_table(self) -> torch.Tensor:
        j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        return (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                2.0 * j / self.rotary_dim)).to(torch.float32)

    def prepare(self, device, dtype) -> None:
        self.inv_freq = self.frequency_table().to(device)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    def __init__(self, head_dim: int = 0, **_) -> None:
        super().__init__()
        self.rotary_dim = 0
        self.interleaved = False
        self.inv_freq = None
