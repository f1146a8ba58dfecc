"""What a layer is made of, in general terms.

A model is a list of *blocks*; a block arranges a *mixer* (attention here), a *feed-forward*
and *norms*; a mixer may use a *position encoding*.  Every part takes its sizes and constants
as constructor arguments and is chosen by the architecture's builder layer by layer, by name,
from the registries below.  No part knows which model it is in: it sees its own parameters and
the ``StepContext`` of the step being run.

Interfaces
----------
``Part``            parameters declared as ``ParamSpec``s (name, shape, init), filled by the loader.
``Mixer``           ``forward(h, ctx, site) -> y``; declares ``cache_spec()`` (paged keys/values)
                    and/or ``state_spec()`` (fixed-size per-request state).
``FeedForward``     ``forward(h, ctx) -> y``.
``Norm``            ``forward(x, pending, out, rows=None)``: adds the pending sub-layer output
                    into the float32 residual stream ``x`` and writes the normalised rows.
``PositionEncoding`` used by a mixer; the rotary one exposes ``inv_freq``/``rotary_dim``/pairing.
``Block``           ``forward(x, pending, ctx, site) -> pending'`` (residual handling is the
                    block's business: pre-norm here).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------ parameters

@dataclass
class ParamSpec:
    """One tensor a part owns.  ``init``: ("normal", std) | ("ones",) | ("ones_jitter", std)."""
    name: str
    shape: Tuple[int, ...]
    init: Tuple = ("normal", 0.02)
    kind: str = "matrix"            # "matrix" | "vector" | "table"


class Part:
    """Base of every part: named parameters, named children.

    ``capturable``: a step that contains the part may be recorded into a CUDA graph and replayed.
    That asks three things of ``forward``: it only enqueues device work (no host synchronisation,
    no host-side reading of device data); everything that changes from step to step reaches it
    through device memory at fixed addresses (the ``StepContext``'s index tensors, the cache, state
    slabs), never through Python values or freshly computed shapes; and a replay does exactly what
    the recorded call did, once -- a part with state of its own may update it in place, the engine
    runs every step exactly once, the step that is recorded included.  A part that cannot promise
    this sets it to False and the engine replays no graphs."""

    capturable = True

    def __init__(self) -> None:
        self._specs: Dict[str, ParamSpec] = {}
        self._params: Dict[str, Optional[torch.Tensor]] = {}
        self._children: Dict[str, "Part"] = {}

    # declaration
    def declare(self, name: str, shape: Sequence[int], init: Tuple = ("normal", 0.02),
                kind: str = "matrix") -> None:
        self._specs[name] = ParamSpec(name, tuple(int(s) for s in shape), init, kind)
        self._params[name] = None

    def add_child(self, name: str, part: "Part") -> "Part":
        self._children[name] = part
        return part

    # access
    def param_specs(self) -> Dict[str, ParamSpec]:
        return dict(self._specs)

    def children(self) -> Dict[str, "Part"]:
        return dict(self._children)

    def set_param(self, name: str, tensor: torch.Tensor) -> None:
        spec = self._specs[name]
        if tuple(tensor.shape) != spec.shape:
            raise ValueError(f"{type(self).__name__}.{name}: shape {tuple(tensor.shape)} != {spec.shape}")
        self._params[name] = tensor
        self.on_param_set(name, tensor)

    def on_param_set(self, name: str, tensor: torch.Tensor) -> None:   # hook for subclasses
        pass

    def param(self, name: str) -> torch.Tensor:
        t = self._params[name]
        if t is None:
            raise RuntimeError(f"{type(self).__name__}.{name} has not been loaded")
        return t

    def named_parts(self, prefix: str = ""):
        yield prefix, self
        for n, c in self._children.items():
            yield from c.named_parts(f"{prefix}.{n}" if prefix else n)

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        """Called once after loading: build device-side constants (tables and the like)."""
        for c in self._children.values():
            c.prepare(device, dtype)


# ----------------------------------------------------------------------------- cache needs

@dataclass(frozen=True)
class CacheSpec:
    """Paged keys and values a mixer needs per layer: geometry and how long keys live."""
    num_kv_heads: int
    head_dim: int
    window: int = 0                 # 0: every key is kept; w: only the last w positions


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state a mixer keeps per layer: one tensor [slots, *shape]."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class LayerCall:
    """One entry of the model's run order: which layer runs, and whose cache it uses.

    ``cache_of``: None = this call site has a cache of its own (and writes it); an integer =
    the index (in the run order) of an earlier call site whose cache it reads without writing."""
    layer: int
    cache_of: Optional[int] = None


# -------------------------------------------------------------------------------- contexts

@dataclass
class GroupView:
    """What a step sees of one layer group: the step's page tables and slot mapping."""
    block_tables: torch.Tensor      # int32 [S, max_blocks]
    slot_mapping: torch.Tensor      # int32 [T]
    block_size: int
    window: int


@dataclass
class SiteCache:
    """The cache of one call site: paged K/V of its layer (a view into the group pool) and/or
    its state slab."""
    group: int = -1
    k: Optional[torch.Tensor] = None        # [pages, nkv, block, hd]
    v: Optional[torch.Tensor] = None
    writes: bool = True
    state: Optional[torch.Tensor] = None    # [slots, *shape]


@dataclass
class StepContext:
    """Everything a part may read about the step being run.  All index tensors are int32 on
    the device; the host-side counts are plain ints."""
    rows: int                        # T (with padding)
    seqs: int                        # S (with padding)
    decode_seqs: int                 # entries [0, decode_seqs) are single rows; rows [0, decode_seqs)
    prefill_rows: int
    prefill_tiles: int
    tile_rows: int
    max_ctx: int
    max_decode_ctx: int
    max_q_len: int
    tokens: torch.Tensor
    positions: torch.Tensor
    row_seq: torch.Tensor
    seq_q_start: torch.Tensor
    seq_q_len: torch.Tensor
    seq_ctx_len: torch.Tensor
    seq_state_slot: torch.Tensor
    tile_seq: torch.Tensor
    tile_q0: torch.Tensor
    logit_rows: torch.Tensor
    groups: List[GroupView]
    dtype: torch.dtype               # storage dtype of activations
    workspace: Any = None            # per-engine scratch provider (see engine.runner.Workspace)
    options: Dict[str, Any] = field(default_factory=dict)


# ------------------------------------------------------------------------------ registries

class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._items: Dict[str, Callable[..., Any]] = {}

    def register(self, name: str, factory: Callable[..., Any] = None, *, replace: bool = False):
        def deco(f):
            if name in self._items and not replace:
                raise ValueError(f"{self.what} '{name}' is already registered")
            self._items[name] = f
            return f
        return deco(factory) if factory is not None else deco

    def get(self, name: str) -> Callable[..., Any]:
        if name not in self._items:
            raise KeyError(f"unknown {self.what} '{name}'; registered: {', '.join(sorted(self._items))}")
        return self._items[name]

    def build(self, name: str, **kwargs):
        return self.get(name)(**kwargs)

    def names(self) -> List[str]:
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")


class Mixer(Part):
    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Block(Part):
    mixer: Mixer

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                site: SiteCache) -> torch.Tensor:
        raise NotImplementedError
