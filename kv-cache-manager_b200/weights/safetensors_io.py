"""Reader and writer for the safetensors container, written against the file format itself:

    8 bytes   little-endian u64  N = length of the JSON header
    N bytes   JSON: {"name": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ...,
                     "__metadata__": {...}}
    rest      raw little-endian tensor bytes; offsets are relative to the end of the header

The reference reads a private flat binary instead (``src/model/weights.cpp:24-83``); reading
the public container by tensor name replaces its Python export step
(``tools/export_weights.py:58-85``).
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
from typing import Dict, Iterable, Iterator, List, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One ``.safetensors`` file, opened, checked and memory-mapped by the C++ core
    (``csrc/core/safetensors.cpp``); tensors are views into the map until copied."""

    def __init__(self, path: str):
        from ..csrc.build import load_core
        self.path = path
        try:
            self._reader = load_core().SafetensorsReader(path)
        except RuntimeError as e:
            raise SafetensorsError(str(e)) from None
        self.metadata = dict(self._reader.metadata())
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int]] = {}
        for name in self._reader.names():
            dtype_name, shape, nbytes = self._reader.info(name)
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has dtype {dtype_name}, which this engine does not read")
            self.entries[name] = (_DTYPES[dtype_name][0], tuple(int(x) for x in shape), int(nbytes))

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the memory map (read-only; copy before changing it).  The
        tensor keeps the map alive."""
        dt, shape, nbytes = self.entries[name]
        if nbytes == 0:
            return torch.empty(shape, dtype=dt)
        buf = (ctypes.c_char * nbytes).from_address(self._reader.address(name))
        buf._map_owner = self._reader                 # the map lives as long as any view of it
        return torch.frombuffer(buf, dtype=dt).reshape(shape)

    def close(self) -> None:
        # Tensors handed out keep the map alive through their buffer; drop only our handle.
        self._reader = None


def open_model_files(folder: str) -> List[SafetensorsFile]:
    """``model.safetensors``, or the shards that ``model.safetensors.index.json`` names."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        shards = sorted(set(wm.values()))
        if not shards:
            raise SafetensorsError(f"{index}: empty weight_map")
        return [SafetensorsFile(os.path.join(folder, s)) for s in shards]
    raise SafetensorsError(f"no model.safetensors (or index) in model folder '{folder}'")


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Writes tensors in the given order.  ``tensors`` is consumed twice, so pass a list or a
    re-iterable; each tensor is made contiguous on the CPU just before it is written."""
    items = list(tensors)
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, t in items:
        if name in header:
            raise SafetensorsError(f"duplicate tensor name '{name}'")
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            c = t.detach().to("cpu").contiguous()
            if c.numel():
                f.write(c.reshape(-1).view(torch.uint8).numpy().data)
    os.replace(tmp, path)
