"""The cache manager.  Host side (C++, ``csrc/core``): page allocator, prefix cache, paged and
contiguous policies behind one interface, page tables per layer group, state slots.  Device
side (``pools.py``): the page pools and state slabs those ids index."""
from ..csrc.build import load_core
from .pools import CachePlan, CachePools, GroupInfo, bytes_per_block, plan_cache

core = load_core()
BlockAllocator = core.BlockAllocator
PrefixCache = core.PrefixCache
PagedManager = core.PagedManager
ContiguousManager = core.ContiguousManager
KVManagerConfig = core.KVManagerConfig
LayerGroupSpec = core.LayerGroupSpec
StateSlots = core.StateSlots
Sequence = core.Sequence
make_kv_manager = core.make_kv_manager


def manager_from_config(kv_cfg, windows=(0,)):
    """A ``KVManager`` from the Python-side ``KVManagerConfig`` dataclass and the groups' windows."""
    c = core.KVManagerConfig()
    c.policy = kv_cfg.policy
    c.num_blocks = int(kv_cfg.num_blocks)
    c.block_size = int(kv_cfg.block_size)
    c.max_seq_len = int(kv_cfg.max_seq_len)
    c.prefix_caching = bool(kv_cfg.prefix_caching) and kv_cfg.policy != "contiguous"
    c.watermark_blocks = int(kv_cfg.watermark_blocks)
    c.watermark_frac = float(kv_cfg.watermark_frac)
    c.groups = [core.LayerGroupSpec(int(w)) for w in windows]
    return core.make_kv_manager(c)


__all__ = ["CachePlan", "CachePools", "GroupInfo", "bytes_per_block", "plan_cache", "core",
           "BlockAllocator", "PrefixCache", "PagedManager", "ContiguousManager", "KVManagerConfig",
           "LayerGroupSpec", "StateSlots", "Sequence", "make_kv_manager", "manager_from_config"]
