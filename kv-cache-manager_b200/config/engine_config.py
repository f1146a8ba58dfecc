"""Engine-side configuration: cache policy, scheduler limits, compute dtype.

Names and defaults follow the reference's structs: ``KVManagerConfig``
(``src/core/kv_manager.h:64-72``), ``SchedulerConfig`` (``src/core/scheduler.h:14-18``) and
``EngineConfig`` (``src/engine/engine.h:16-22``).  Added here: the compute dtype, the prefill
portion cap, sampling seed and the number of fixed-size state slots.
"""
from __future__ import annotations

from dataclasses import dataclass, field

DTYPE_ALIASES = {
    "bf16": "bfloat16", "bfloat16": "bfloat16",
    "fp32": "float32", "float32": "float32", "f32": "float32",
}


def canonical_dtype(name: str) -> str:
    try:
        return DTYPE_ALIASES[name.lower()]
    except KeyError:
        raise ValueError(f"unknown dtype '{name}'; use bfloat16 or float32") from None


@dataclass
class KVManagerConfig:
    policy: str = "paged"            # "paged" | "contiguous"
    num_blocks: int = 1024           # <= 0: derived from EngineConfig.pool_gb
    block_size: int = 16
    max_seq_len: int = 2048
    prefix_caching: bool = False
    watermark_blocks: int = -1       # paged: blocks kept spare at admission (-1: watermark_frac)
    watermark_frac: float = 0.01


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256          # cap on the running batch
    max_batched_tokens: int = 4096   # cap on rows computed per step (prompt portions + decodes)
    prefill_chunk: int = 0           # cap on one request's prompt portion per step (0: budget only)
    chunked_prefill: bool = True     # False: a prompt is only ever scheduled whole


@dataclass
class EngineConfig:
    kv: KVManagerConfig = field(default_factory=KVManagerConfig)
    pool_gb: float = 1.0
    sched: SchedulerConfig = field(default_factory=SchedulerConfig)
    dtype: str = "bfloat16"
    attn: str = "auto"               # decode attention: "v1" (whole context) | "v2" (split) | "auto"
    gemm: str = "auto"               # bfloat16 products: "auto" (fastest measured: this engine's kernels or the
                                     # library) | "native" (this engine's kernels only) | "library" | "plain"
    max_logit_rows: int = 0          # 0: max(max_num_seqs, 512)
    sampling_seed: int = 0
    eos_token_id: int = -1           # < 0: no end-of-sequence stop (the reference has none)
    cuda_graphs: bool = True         # capture decode-only steps per batch-size bucket
    native_loop: bool = True         # run the request loop and the layer loop in C++ where the model allows it
    fuse_norms: bool = True          # steps of at most 8 rows: residual add and norms inside the streaming products
    lookahead: bool = True           # C++ loop: enqueue the next greedy decode step before this one's tokens are read
    device: str = "cuda:0"
