"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference keeps the same facts in a 64-byte binary header (``src/model/weights.cpp:24-40``)
that its export script fills from the HF config (``tools/export_weights.py:59-67``); here the
JSON is read directly.  Every size and constant a layer needs comes from this object: parts
take them as constructor parameters and never read a config themselves.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields, asdict
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: names the key and the reason."""


def _require(d: Dict[str, Any], key: str, typ, where: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"{where}: required key '{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{where}: key '{key}' must be an integer, got {v!r}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
    return v


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration; subclasses add their own keys."""
    architecture: str

    def to_json_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """Llama dense decoder (``LlamaForCausalLM``).

    Field <- config.json key, as the reference maps them (``src/model/weights.h:12-18``,
    ``tools/export_weights.py:59-67``).  ``head_dim`` is the key of that name when present and
    ``hidden_size // num_attention_heads`` otherwise (the reference computes the latter at
    export, ``tools/export_weights.py:62``); it need not equal ``hidden_size / heads`` here.
    """
    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    max_position_embeddings: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"

    # ---- derived sizes
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def validate(self) -> None:
        w = "LlamaConfig"
        for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim",
                  "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"{w}: '{f}' must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"{w}: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"{w}: head_dim ({self.head_dim}) must be even for rotary pairs")
        if self.hidden_act != "silu":
            raise ConfigError(f"{w}: hidden_act '{self.hidden_act}' is not supported (only 'silu')")
        if not (self.rope_theta > 0):
            raise ConfigError(f"{w}: rope_theta must be positive, got {self.rope_theta}")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"{w}: rms_norm_eps must be positive, got {self.rms_norm_eps}")

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        w = "config.json (LlamaForCausalLM)"
        heads = _require(d, "num_attention_heads", int, w)
        hidden = _require(d, "hidden_size", int, w)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{w}: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        # rotary base: plain key, or the nested form newer exports use
        rope_params = d.get("rope_parameters") or {}
        theta = d.get("rope_theta", rope_params.get("rope_theta", 10000.0))
        scaling = d.get("rope_scaling")
        if scaling is None and rope_params.get("rope_type", "default") not in ("default", None):
            scaling = rope_params
        if scaling not in (None, {}):
            rt = scaling.get("rope_type", scaling.get("type", "?")) if isinstance(scaling, dict) else scaling
            if rt != "default":
                raise ConfigError(f"{w}: rope scaling '{rt}' is not supported (plain rotary only)")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"{w}: '{key}' = true is not supported (no bias tensors)")
        if d.get("sliding_window") not in (None, 0):
            raise ConfigError(f"{w}: 'sliding_window' is not part of this architecture")
        cfg = cls(
            architecture="LlamaForCausalLM",
            vocab_size=_require(d, "vocab_size", int, w),
            hidden_size=hidden,
            intermediate_size=_require(d, "intermediate_size", int, w),
            num_hidden_layers=_require(d, "num_hidden_layers", int, w),
            num_attention_heads=heads,
            num_key_value_heads=int(d.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            max_position_embeddings=_require(d, "max_position_embeddings", int, w),
            rope_theta=float(theta),
            rms_norm_eps=_require(d, "rms_norm_eps", float, w),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
        )
        cfg.validate()
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d.pop("architecture")
        d["architectures"] = [self.architecture]
        d["model_type"] = "llama"
        return d


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder '{folder}'")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return d
