"""Fills a model's parameters from safetensors by tensor name.

dtype rule: with a bfloat16 engine, tensors stored in 16 bits (BF16, F16) are kept as bfloat16,
integer tensors become int32, and a tensor stored in 32 bits stays float32 (its part then
computes with it in float32).  With a float32 engine every floating tensor becomes float32.

All problems of a checkpoint are reported in ONE ``WeightError``: tensors that are missing,
tensors with a wrong shape, and tensors the model has no use for.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..models.spec import ModelSpec, TensorBinding
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files


class WeightError(ValueError):
    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str],
                 where: str) -> None:
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"weights in '{where}' do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        super().__init__("\n".join(lines))


def target_dtype(stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return engine_dtype


class _Source:
    """Name -> tensor over one or several files, or over an in-memory dict."""

    def __init__(self, files: Optional[List[SafetensorsFile]] = None,
                 tensors: Optional[Dict[str, torch.Tensor]] = None) -> None:
        self.files = files or []
        self.tensors = tensors or {}
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self.where[n] = f

    def names(self) -> List[str]:
        return list(self.where) + list(self.tensors)

    def shape(self, name: str) -> Optional[Tuple[int, ...]]:
        if name in self.tensors:
            return tuple(self.tensors[name].shape)
        if name in self.where:
            return self.where[name].info(name)[1]
        return None

    def get(self, name: str) -> torch.Tensor:
        return self.tensors[name] if name in self.tensors else self.where[name].tensor(name)


def _place(binding: TensorBinding, src: _Source, device, engine_dtype) -> torch.Tensor:
    pieces = []
    for name, _ in binding.sources:
        t = src.get(name)
        pieces.append(t.to(device=device, dtype=target_dtype(t.dtype, engine_dtype)))
    if len(pieces) == 1:
        return pieces[0].contiguous()
    if len({p.dtype for p in pieces}) != 1:                  # mixed storage: widest wins
        pieces = [p.to(torch.float32) for p in pieces]
    return torch.cat(pieces, dim=0).contiguous()


def load_into(spec: ModelSpec, src: _Source, device, engine_dtype: torch.dtype, where: str) -> None:
    missing: List[str] = []
    wrong: List[str] = []
    used = set()
    use_tie: Dict[int, bool] = {}
    for i, b in enumerate(spec.bindings):
        present = [src.shape(n) is not None for n, _ in b.sources]
        if b.tie_to is not None and (b.tied or not any(present)):
            use_tie[i] = True
            used.update(n for n, _ in b.sources)              # a stored copy of a tied tensor is ignored
            continue
        for (n, want), ok in zip(b.sources, present):
            if not ok:
                missing.append(n)
                continue
            used.add(n)
            got = src.shape(n)
            if tuple(got) != tuple(want):
                wrong.append(f"{n}: file has {list(got)}, model needs {list(want)}")
    unexpected = sorted(n for n in src.names()
                        if n not in used and not any(s in n for s in spec.ignorable))
    if missing or wrong or unexpected:
        raise WeightError(sorted(missing), unexpected, wrong, where)
    placed: Dict[int, torch.Tensor] = {}
    for i, b in enumerate(spec.bindings):
        if use_tie.get(i):
            continue
        placed[id(b)] = _place(b, src, device, engine_dtype)
        b.part.set_param(b.param, placed[id(b)])
    for i, b in enumerate(spec.bindings):
        if use_tie.get(i):
            b.part.set_param(b.param, placed[id(b.tie_to)])   # the same storage, not a copy
    for _, part in spec.parts():
        part.prepare(torch.device(device), engine_dtype)


def load_weights(spec: ModelSpec, folder: str, device, engine_dtype: torch.dtype) -> None:
    """Reads ``folder/model.safetensors`` (or its shards) into the model's parts."""
    files = open_model_files(folder)
    try:
        load_into(spec, _Source(files=files), device, engine_dtype, folder)
    finally:
        for f in files:
            f.close()


def load_from_tensors(spec: ModelSpec, tensors: Dict[str, torch.Tensor], device,
                      engine_dtype: torch.dtype) -> None:
    """The same checks and placement for tensors that are already in memory."""
    load_into(spec, _Source(tensors=tensors), device, engine_dtype, "<memory>")
