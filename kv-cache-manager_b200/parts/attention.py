"""Grouped-query attention over the paged cache: the mixer of this architecture.

Per step: fused QKV product; rotary encoding of q and k in place and the write of K (encoded)
and V into the rows' page slots (one kernel); attention of every row over its request's pages
(keys up to the row's own position, optionally only the last ``window`` of them); output
product.  Order and formulas after ``src/model/llama.cpp:108-116``; scale = 1/sqrt(head_dim)
unless given.  All rows of a step are written to the cache before any row reads it, so rows of
one portion see each other through the pages and causality is the bound ``position + 1``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import library as K
from .base import CacheSpec, MIXERS, Mixer, PositionEncoding, SiteCache, StepContext
from .linear import Linear


@MIXERS.register("attention")
class PagedAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PositionEncoding, window: int = 0, scale: Optional[float] = None) -> None:
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        self.hidden, self.nh, self.nkv, self.hd = hidden, num_heads, num_kv_heads, head_dim
        self.window = int(window or 0)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = self.add_child("position", position)
        self.qkv = self.add_child("qkv", Linear(hidden, (num_heads + 2 * num_kv_heads) * head_dim))
        self.o = self.add_child("o", Linear(num_heads * head_dim, hidden))

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.nkv, self.hd, self.window)

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        g = ctx.groups[site.group]
        pos = self.position
        w = self.qkv.param("weight")
        M = h.shape[0]
        # A handful of rows (decode): one kernel does the product, the rotary encoding and the
        # cache write; it gives the same bits as the three separate kernels below.
        if (site.writes and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and ctx.options.get("gemm", "auto") in ("auto", "native") and ctx.options.get("fuse", True)
                and pos.inv_freq is not None and pos.rotary_dim == self.hd and not pos.interleaved
                and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
                and K.qkv_rope_cache_supported(M, h.shape[1], self.nh, self.nkv, self.hd)):
            qkv = torch.empty((M, self.nh * self.hd), dtype=h.dtype, device=h.device)
            K.qkv_rope_cache(h, w, qkv, ctx.positions, pos.inv_freq, g.slot_mapping, site.k, site.v,
                             self.nh, self.nkv, self.hd)
        else:
            qkv = self.qkv.forward(h, ctx)
            K.rope_cache(qkv, ctx.positions, pos.inv_freq, pos.rotary_dim, pos.interleaved,
                         g.slot_mapping, site.k, site.v, self.nh, self.nkv, self.hd, g.block_size,
                         write_cache=site.writes)
        out = torch.empty((h.shape[0], self.nh * self.hd), dtype=h.dtype, device=h.device)
        K.paged_attention(qkv, out, site.k, site.v, g.block_tables, ctx, self.nh, self.nkv, self.hd,
                          self.scale, self.window)
        return self.o.forward(out, ctx)
