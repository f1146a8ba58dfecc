"""From a model folder to a model with loaded parts."""
from __future__ import annotations

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.engine_config import canonical_dtype
from ..config.registry import get_architecture, load_config
from ..models.spec import ModelSpec
from ..weights.loader import load_from_tensors, load_weights

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def torch_dtype(name: str) -> torch.dtype:
    return TORCH_DTYPES[canonical_dtype(name)]


def load_model(folder: str, dtype: str = "bfloat16", device="cuda:0") -> ModelSpec:
    """config.json -> architecture -> parts; model.safetensors -> their parameters."""
    cfg = load_config(folder)
    spec = get_architecture(cfg.architecture).build(cfg)
    load_weights(spec, folder, device, torch_dtype(dtype))
    return spec


def model_from_tensors(cfg, tensors, dtype: str = "bfloat16", device="cuda:0") -> ModelSpec:
    spec = get_architecture(cfg.architecture).build(cfg)
    load_from_tensors(spec, dict(tensors), device, torch_dtype(dtype))
    return spec
