"""Random-weights mode: a model folder (config.json + model.safetensors) from a configuration
and a seed.  Matrices and tables N(0, std) (std from the part's declaration, 0.02 by default),
norm weights 1, or 1 + N(0, jitter) when asked.  Each tensor's stream is seeded by
(seed, tensor name), so values do not depend on the order of generation."""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from ..config.registry import get_architecture
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(config, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                   norm_jitter: float = 0.0) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (checkpoint name, tensor) for every tensor the architecture reads.  A tied output
    head is not written (it falls back to the embedding at load)."""
    spec = get_architecture(config.architecture).build(config)
    for b in spec.bindings:
        if b.tie_to is not None and b.tied:
            continue
        init = b.part.param_specs()[b.param].init
        for name, shape in b.sources:
            g = torch.Generator(device=device)
            g.manual_seed(_tensor_seed(seed, name))
            if init[0] == "normal":
                t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * init[1]
            elif init[0] in ("ones", "ones_jitter"):
                t = torch.ones(shape, device=device, dtype=torch.float32)
                jitter = norm_jitter if init[0] == "ones" else init[1]
                if jitter:
                    t = t + torch.randn(shape, generator=g, device=device, dtype=torch.float32) * jitter
            else:
                raise ValueError(f"unknown init {init!r} for {name}")
            yield name, t.to(dtype)


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       norm_jitter: float = 0.0) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        d = config.to_json_dict()
        d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                            torch.float16: "float16"}[dtype]
        json.dump(d, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      list(random_tensors(config, seed, dtype, "cpu", norm_jitter)),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
