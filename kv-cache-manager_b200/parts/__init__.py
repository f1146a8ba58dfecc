"""Layer parts: mixers, feed-forwards, norms, position encodings, blocks (see ``base.py``)."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec,
                   FeedForward, GroupView, LayerCall, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding, Registry, SiteCache, StateSpec, StepContext)
from .linear import Linear, matmul_nt
from .norm import RMSNorm
from .rope import NoPositionEncoding, RotaryEmbedding
from .attention import PagedAttention
from .mlp import GatedMLP
from .embedding import Embedding, LMHead
from .block import PreNormBlock

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheSpec",
    "FeedForward", "GroupView", "LayerCall", "Mixer", "Norm", "ParamSpec", "Part",
    "PositionEncoding", "Registry", "SiteCache", "StateSpec", "StepContext", "Linear", "matmul_nt",
    "RMSNorm", "NoPositionEncoding", "RotaryEmbedding", "PagedAttention", "GatedMLP", "Embedding",
    "LMHead", "PreNormBlock",
]
