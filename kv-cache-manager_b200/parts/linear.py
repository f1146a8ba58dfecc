"""Matrix product of a part: y = x W^T with W stored [out_features, in_features] (no bias), the
layout of every matrix of the reference (``src/model/llama.cpp:45-52``).

Which kernel runs is decided by the weight's dtype, never by the model:
* float32 weight  -> this engine's plain float kernel (true 32-bit, fixed summation order);
* bfloat16 weight -> this engine's weight-streaming kernel for a handful of rows (decode), else
  the library GEMM (cuBLAS through ``torch.mm``, the same place where the reference calls cuBLAS);
  this engine's tcgen05 kernels for many rows on request, and for the fused gate/up product;
  ``options['gemm']``: 'plain' forces the plain twin, 'library' cuBLAS, 'tcgen05' and 'pair'
  the respective kernels; 'native' never calls the library: the streaming kernel up to 16 rows, the
  split-K tcgen05 kernel up to 255, from 256 the tiled tcgen05 kernel (one SM per tile) or, for wide
  outputs, its two-SM form (slower than 'auto' where 'auto' takes the library: 17 to 255 rows, and
  tile counts that fill the SMs badly).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import Part, StepContext


STREAM_MAX_BYTES = 32 << 20
TCGEN05_MIN_ROWS = 256
TCGEN05_GATED_MAX_HIDDEN = 3072    # beyond, the library product plus the activation kernel is faster
PAIR_MIN_COLS = 8192               # from here the two-SM tcgen05 kernel is faster than the one-SM kernel


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
    # A handful of rows (decode): this engine's weight-streaming kernel.  Measured on B200 at 8 rows
    # it beats the library (4-7 us against 7-16 us at 8-23 MB) or ties it (46 and 131 MB); from 9
    # to 16 rows the library streams matrices beyond STREAM_MAX_BYTES faster.
    native = mode == "native"
    if mode != "library" and (native or M <= 8 or w.numel() * 2 <= STREAM_MAX_BYTES) and K.stream_gemm_supported(M, N, w.shape[1]) \
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        K.gemm_stream(x, w, y)
        return y
    # Many rows (prefill): this engine's tiled tcgen05 kernel with 'tcgen05' or 'native'.  'auto'
    # takes the library here: measured at 2,048 rows its kernels are 10-25 % faster for a plain
    # product (2048 x 2048: 16.4 against 18.8 us, 2048 x 5632: 35.4 against 40.6 us; a Llama-3-8B
    # shaped prefill: 27 against 34 ms); the tcgen05 kernel earns its place in 'auto' where it
    # saves a kernel: the gate/up product with the activation in its epilogue (parts/mlp.py).
    if mode == "pair" or (native and M >= TCGEN05_MIN_ROWS and N >= PAIR_MIN_COLS):
        if K.pair_gemm_supported(x, w):
            y = torch.empty((M, N), dtype=out_dtype, device=x.device)
            K.gemm_tcgen05_pair(x, w, y)
            return y
    if mode == "tcgen05" or (native and M >= TCGEN05_MIN_ROWS):
        if K.tcgen05_gemm_supported(x, w):
            y = torch.empty((M, N), dtype=out_dtype, device=x.device)
            K.gemm_tcgen05(x, w, y)
            return y
    # In between: the library, unless the caller wants this engine's kernels only (the split-K
    # tcgen05 kernel: correct and reproducible, about half the library's speed at these sizes).
    if (native or mode == "splitk") and K.splitk_gemm_supported(x, w):
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        K.gemm_tcgen05_splitk(x, w, y)
        return y
    y = torch.mm(x, w.t()) if out_dtype == torch.bfloat16 else torch.mm(x, w.t(), out_dtype=out_dtype)
    K.profile_mark("library_gemm")
    return y


def tiles_fill_well(M: int, N: int, device) -> bool:
    """The tcgen05 kernel's 128 x 256 tiles give every SM work in every round but (at most a fifth
    of) the last."""
    sms = K.sm_count(device)
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    rounds = (tiles + sms - 1) // sms
    return tiles >= sms and tiles >= 0.8 * rounds * sms
