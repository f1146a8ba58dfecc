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

import json
import mmap
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
    """Memory-maps one ``.safetensors`` file; tensors are views into the map until copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open '{path}': {e.strerror}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8 or n > (100 << 20):
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt, isz = _DTYPES[e["dtype"]]
                shape = tuple(int(x) for x in e["shape"])
                b, en = (int(x) for x in e["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: bad header entry for '{name}': {e!r}") from None
            numel = 1
            for s in shape:
                numel *= s
            if b < 0 or en < b or en > data_len:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' data_offsets [{b}, {en}) lie outside the data "
                    f"section of {data_len} bytes (file truncated?)")
            if en - b != numel * isz:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' has {en - b} bytes but shape {list(shape)} of "
                    f"{e['dtype']} needs {numel * isz}")
            self.entries[name] = (dt, shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the memory map (read-only; copy before changing it)."""
        dt, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._mm)[self._data_start + b:self._data_start + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")       # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=dt)
        return t.reshape(shape)

    def close(self) -> None:
        # Tensors handed out keep the map alive through their buffer; drop only our handles.
        self._mm = None
        self._f.close()


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
