"""What an architecture's builder returns: the parts of one model, the order in which its layers
run, and how its parameters map to checkpoint tensor names."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence, Tuple

from ..parts.base import Block, LayerCall, Part


@dataclass
class TensorBinding:
    """Parameter ``param`` of ``part`` = the listed checkpoint tensors concatenated along dim 0
    (one name for a plain tensor; q,k,v or gate,up for a fused matrix).

    ``tie_to``: another binding whose tensor is used instead when ``tied`` is set or when the
    checkpoint lacks the sources (the reference's export falls back the same way for the output
    head, ``tools/export_weights.py:82``)."""
    part: Part
    param: str
    sources: List[Tuple[str, Tuple[int, ...]]]
    tie_to: Optional["TensorBinding"] = None
    tied: bool = False


@dataclass
class ModelSpec:
    config: Any
    embedding: Part
    blocks: List[Block]
    order: List[LayerCall]
    final_norm: Part
    lm_head: Part
    bindings: List[TensorBinding] = field(default_factory=list)
    ignorable: Sequence[str] = ()          # substrings of checkpoint names that may be skipped

    def parts(self):
        yield "embedding", self.embedding
        for i, b in enumerate(self.blocks):
            yield f"blocks.{i}", b
        yield "final_norm", self.final_norm
        yield "lm_head", self.lm_head
