"""Reading and writing the safetensors container, without a third-party reader.

Layout: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the raw little-endian tensor data.  Tensors are read lazily from a memory map,
one at a time by name, as the reference reads GGUF tensors on demand
(src/io/gguf_reader.cpp:410-423).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

from ..errors import CitlaliError, require

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def dtype_name(dtype: torch.dtype) -> str:
    require(dtype in _NAMES, f"dtype {dtype} cannot be stored in safetensors by this writer")
    return _NAMES[dtype]


class SafetensorsFile:
    """One ``.safetensors`` file: a directory of tensors and a memory map of their bytes."""

    def __init__(self, path: str):
        self.path = path
        require(os.path.isfile(path), f"no such weights file: {path}")
        size = os.path.getsize(path)
        require(size >= 8, f"{path}: too short to be a safetensors file")
        self._file = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        require(8 + header_len <= size, f"{path}: header length {header_len} exceeds the file size {size}")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CitlaliError(f"{path}: the header is not valid JSON ({e})") from None
        require(isinstance(header, dict), f"{path}: the header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + header_len
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dt, shape, (begin, end) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise CitlaliError(f"{path}: malformed header entry for tensor '{name}'") from None
            require(dt in _DTYPES, f"{path}: tensor '{name}' has dtype {dt}, which is not implemented")
            count = 1
            for s in shape:
                count *= s
            itemsize = torch.empty((), dtype=_DTYPES[dt]).element_size()
            require(end - begin == count * itemsize and 0 <= begin <= end and self._data_start + end <= size,
                    f"{path}: tensor '{name}' has data offsets [{begin}, {end}) that do not fit shape "
                    f"{list(shape)} of {dt} in a file of {size} bytes")
            self._entries[name] = (dt, shape, begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name][0]]

    def read(self, name: str) -> torch.Tensor:
        """A host tensor that owns its memory (a copy out of the map)."""
        require(name in self._entries, f"{self.path}: no tensor named '{name}'")
        dt, shape, begin, end = self._entries[name]
        dtype = _DTYPES[dt]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        flat = torch.from_numpy(np.frombuffer(view, dtype=np.uint8).copy())
        return flat.view(dtype).reshape(shape)

    def view(self, name: str) -> torch.Tensor:
        """The tensor as it lies in the memory map: no copy, read-only, valid until :meth:`close`."""
        import warnings
        require(name in self._entries, f"{self.path}: no tensor named '{name}'")
        dt, shape, begin, end = self._entries[name]
        dtype = _DTYPES[dt]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")            # torch warns that the buffer cannot be written; it is only read
            flat = torch.from_numpy(np.frombuffer(view, dtype=np.uint8))
        return flat.view(dtype).reshape(shape)

    def close(self):
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass            # a view of the map is still alive somewhere; the map goes when it does
            self._map = None
        self._file.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None):
    """Write ``(name, tensor)`` pairs.  ``tensors`` may be a generator that is run twice
    through a callable: pass a list for small models, or a ``lambda: iterator`` so that a
    large model is produced tensor by tensor without holding all of it."""
    produce = tensors if callable(tensors) else (lambda: iter(list(tensors)))
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    seen = set()
    for name, t in produce():
        require(name not in seen, f"tensor '{name}' given twice to the safetensors writer")
        seen.add(name)
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": dtype_name(t.dtype), "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".partial"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, t in produce():
            t = t.detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
