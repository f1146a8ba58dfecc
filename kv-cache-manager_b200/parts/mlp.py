"""Gated feed-forward: down( act(x Wg^T) * (x Wu^T) ), gate and up fused into one matrix
[2I, H] (gate rows first) so that one product feeds the activation kernel
(``src/model/llama.cpp:120-122``; activation ``src/cuda/kernels.cu:72-82``).
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import FEED_FORWARDS, FeedForward, StepContext
from .linear import Linear, TCGEN05_GATED_MAX_HIDDEN, TCGEN05_MIN_ROWS, tiles_fill_well


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, hidden: int, intermediate: int, activation: str = "silu") -> None:
        super().__init__()
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation '{activation}' has no kernel (only 'silu')")
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up = self.add_child("gate_up", Linear(hidden, 2 * intermediate))
        self.down = self.add_child("down", Linear(intermediate, hidden))

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = torch.empty((h.shape[0], self.intermediate), dtype=h.dtype, device=h.device)
        w = self.gate_up.param("weight")
        # A handful of rows (decode): the gate/up product and the activation in one kernel (the
        # same roundings as the two separate kernels).
        if (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ctx.options.get("gemm", "auto") in ("auto", "native")
                and ctx.options.get("fuse", True) and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
                and K.gate_up_silu_supported(h.shape[0], self.intermediate, h.shape[1])):
            K.gate_up_silu(h, w, act)
        elif (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ctx.options.get("fuse", True)
              and ctx.options.get("gemm", "auto") in ("auto", "native", "tcgen05", "pair") and h.shape[0] >= TCGEN05_MIN_ROWS
              and (ctx.options.get("gemm", "auto") != "auto"
                   or (tiles_fill_well(h.shape[0], 2 * self.intermediate, h.device)
                       and h.shape[1] <= TCGEN05_GATED_MAX_HIDDEN))
              and K.tcgen05_gemm_supported(h, w)):
            # Many rows (prefill): the tcgen05 product applies the activation in its epilogue.  It
            # saves the activation kernel (time ~ rows x I) and loses about a tenth of the product
            # against the library (time ~ rows x I x hidden): a win up to a hidden size of ~3,000
            # (TinyLlama shape: 84 us against 76 + 15; Llama-3-8B shape: the library wins).
            # Beyond that size the two-SM form of the kernel is the faster of this engine's two
            # (Llama-3-8B shape: about 0.4 against 0.58 ms).
            if ctx.options.get("gemm", "auto") == "pair" or h.shape[1] > TCGEN05_GATED_MAX_HIDDEN:
                K.gate_up_silu_tcgen05_pair(h, w, act)
            else:
                K.gate_up_silu_tcgen05(h, w, act)
        else:
            K.silu_mul(self.gate_up.forward(h, ctx), act)
        return self.down.forward(act, ctx)
