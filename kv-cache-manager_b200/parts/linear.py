"""Matrix product of a part: y = x W^T with W stored [out_features, in_features] (no bias), the
layout of every matrix of the reference (``src/model/llama.cpp:45-52``).

Which kernel runs is decided by the weight's dtype, never by the model:
* float32 weight  -> this engine's plain float kernel (true 32-bit, fixed summation order);
* bfloat16 weight -> the library GEMM (cuBLAS through ``torch.mm``), the same place where the
  reference calls cuBLAS, or this engine's own weight-streaming kernel for a handful of rows
  (decode), or the plain kernel when ``options['gemm'] == 'plain'`` asks for the twin
  (``'library'`` forces cuBLAS, ``'skinny'`` the register-streaming variant).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import Part, StepContext


STREAM_MAX_BYTES = 32 << 20


class Linear(Part):
    def __init__(self, in_features: int, out_features: int, init_std: float = 0.02) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.declare("weight", (out_features, in_features), ("normal", init_std), "matrix")

    def forward(self, x: torch.Tensor, ctx: Optional[StepContext] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        w = self.param("weight")
        return matmul_nt(x, w, out_dtype or x.dtype, (ctx.options if ctx is not None else {}))


def matmul_nt(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, options: dict) -> torch.Tensor:
    """x [M,K] times w [N,K] transposed -> [M,N] in ``out_dtype``."""
    M = x.shape[0]
    N = w.shape[0]
    if w.dtype == torch.float32:
        xin = x if x.dtype == torch.float32 else x.float()
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        K.gemm_plain(xin, w, y)
        return y if out_dtype == torch.float32 else y.to(out_dtype)
    if w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        raise K.KernelError(f"matmul: unsupported operand dtypes {x.dtype} x {w.dtype}")
    mode = options.get("gemm", "auto")
    if mode == "plain":
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        K.gemm_plain(x, w, y)
        return y
    if mode == "skinny" and K.skinny_gemm_supported(M, N, w.shape[1]):
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        K.gemm_skinny(x, w, y)
        return y
    # A handful of rows (decode): this engine's weight-streaming kernel, for matrices up to
    # STREAM_MAX_BYTES; measured on B200 it beats the library there (5-10 us against 7-15 us at
    # 8-23 MB) while the library's kernels stream the largest matrices (46-131 MB) faster.
    if mode != "library" and w.numel() * 2 <= STREAM_MAX_BYTES and K.stream_gemm_supported(M, N, w.shape[1]) \
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        K.gemm_stream(x, w, y)
        return y
    if out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)
