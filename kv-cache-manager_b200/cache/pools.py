"""Device side of the cache: page pools per layer group and state slabs per call site.

A *call site* is one entry of the model's run order.  Sites whose mixers ask for paged keys and
values with the same geometry and window form a *layer group*: one pool
``[sites, pages, kv heads, page size, head dim]`` for K and one for V (a page id addresses the
same page in every site of its group, as in the reference's per-layer pools,
``src/cuda/kv_cache.h:1-2``), and one page table per request.  Pools are zero-filled so that a
stray read is deterministic (``src/cuda/kv_cache.cu:12-14``).  Sites whose mixers ask for
fixed-size state get a slab ``[slots, *shape]`` indexed by the request's state slot.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import CacheSpec, SiteCache, StateSpec


@dataclass
class GroupInfo:
    spec: CacheSpec
    sites: List[int] = field(default_factory=list)     # run-order indices that own a layer of the pool


@dataclass
class CachePlan:
    """Which call site uses which group/layer of the pools; derived from the model alone."""
    groups: List[GroupInfo]
    site_group: List[int]            # per call site: group index or -1
    site_layer: List[int]            # per call site: index inside the group's pool
    site_writes: List[bool]
    site_state: List[Optional[StateSpec]]

    @property
    def windows(self) -> List[int]:
        return [g.spec.window for g in self.groups]

    @property
    def has_state(self) -> bool:
        return any(s is not None for s in self.site_state)


def plan_cache(spec) -> CachePlan:
    groups: List[GroupInfo] = []
    key_to_group: Dict[CacheSpec, int] = {}
    n = len(spec.order)
    site_group, site_layer, site_writes = [-1] * n, [-1] * n, [True] * n
    site_state: List[Optional[StateSpec]] = [None] * n
    for k, call in enumerate(spec.order):
        mixer = spec.blocks[call.layer].mixer
        cs, ss = mixer.cache_spec(), mixer.state_spec()
        if call.cache_of is not None:
            src = call.cache_of
            if not (0 <= src < k) or spec.order[src].cache_of is not None:
                raise ValueError(f"run order entry {k}: cache_of must name an earlier entry that owns a cache")
            src_spec = spec.blocks[spec.order[src].layer].mixer.cache_spec()
            if cs is None or src_spec != cs:
                raise ValueError(f"run order entry {k}: cannot read the cache of entry {src} "
                                 f"({src_spec}) with a mixer that needs {cs}")
            site_group[k], site_layer[k], site_writes[k] = site_group[src], site_layer[src], False
        elif cs is not None:
            if cs not in key_to_group:
                key_to_group[cs] = len(groups)
                groups.append(GroupInfo(cs))
            g = key_to_group[cs]
            site_group[k], site_layer[k] = g, len(groups[g].sites)
            groups[g].sites.append(k)
        site_state[k] = ss
    return CachePlan(groups, site_group, site_layer, site_writes, site_state)


class CachePools:
    def __init__(self, plan: CachePlan, num_blocks: int, block_size: int, num_slots: int,
                 dtype: torch.dtype, device) -> None:
        self.plan, self.num_blocks, self.block_size, self.num_slots = plan, num_blocks, block_size, num_slots
        self.dtype = dtype
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        for g in plan.groups:
            shape = (len(g.sites), num_blocks, g.spec.num_kv_heads, block_size, g.spec.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=device))
        self.state: List[Optional[torch.Tensor]] = [
            None if s is None else torch.zeros((num_slots, *s.shape), dtype=s.dtype, device=device)
            for s in plan.site_state]
        self.sites: List[SiteCache] = []
        for k in range(len(plan.site_group)):
            g = plan.site_group[k]
            self.sites.append(SiteCache(
                group=g, k=self.k[g][plan.site_layer[k]] if g >= 0 else None,
                v=self.v[g][plan.site_layer[k]] if g >= 0 else None,
                writes=plan.site_writes[k], state=self.state[k]))

    def reset_slot(self, slot: int) -> None:
        """A request that starts (again) from its first token starts from zero state."""
        for s in self.state:
            if s is not None:
                s[slot].zero_()

    def total_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)


def bytes_per_block(plan: CachePlan, block_size: int, dtype: torch.dtype) -> int:
    """K and V of one page id across every site of every group (``src/cuda/kv_cache.h:20-23``)."""
    item = torch.empty((), dtype=dtype).element_size()
    return sum(2 * len(g.sites) * g.spec.num_kv_heads * block_size * g.spec.head_dim * item
               for g in plan.groups)
