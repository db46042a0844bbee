"""Binding tensors by name: ``WeightLoader`` reads a model folder, ``WeightHandle`` is what
model code sees.

The reference's loader finds a tensor by its GGUF name, converts it and uploads it
(include/citlali/model/weight_loader.h:20-61, src/model/weight_loader.cpp:377-467) and the
model checks every shape at load (src/model/qwen_model.cpp:29-34, :156-173), failing on the
first problem.  Here the names are the checkpoint's own (HF) names, the stored dtype is
kept (bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, integer tables become
int32), and all problems of a folder are reported together in one error.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import CitlaliError, require
from .safetensors_io import SafetensorsFile

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects: checkpoint name, shape, and what it is (``matrix``: [out, in]
    of a linear map or an embedding table; ``gain``: a norm's scale; ``state``: other
    floating-point parameters; ``table``: integers)."""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclass
class WeightHandle:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    tensor: torch.Tensor

    @property
    def out_features(self) -> int:      # rows of an [out, in] matrix (weight_loader.h:29-32)
        return self.shape[0]

    @property
    def in_features(self) -> int:
        return self.shape[1]

    @property
    def nbytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def _kept_dtype(stored: torch.dtype, role: str) -> Optional[torch.dtype]:
    """The dtype a stored tensor is kept in; ``None`` if the stored dtype cannot serve the role."""
    if role == "table":
        return torch.int32 if stored in _INTS else None
    if stored in (torch.float32, torch.float64):
        return torch.float32
    if stored in (torch.bfloat16, torch.float16):
        return torch.bfloat16
    return None


class WeightLoader:
    """Opens the safetensors file(s) of a model folder and hands out tensors by name."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        index_path = os.path.join(model_dir, INDEX_FILE)
        single_path = os.path.join(model_dir, SINGLE_FILE)
        if os.path.isfile(single_path):
            paths = [single_path]
        elif os.path.isfile(index_path):
            with open(index_path, "r", encoding="utf-8") as f:
                index = json.load(f)
            require(isinstance(index.get("weight_map"), dict), f"{index_path}: no 'weight_map' object")
            paths = [os.path.join(model_dir, p) for p in sorted(set(index["weight_map"].values()))]
        else:
            raise CitlaliError(f"no {SINGLE_FILE} (or {INDEX_FILE}) in model folder '{model_dir}'")
        for p in paths:
            f = SafetensorsFile(p)
            self._files.append(f)
            for name in f.names():
                require(name not in self._where, f"tensor '{name}' appears in more than one weights file")
                self._where[name] = f

    def names(self) -> List[str]:
        return list(self._where)

    def has(self, name: str) -> bool:
        return name in self._where

    def stored_shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].shape(name)

    def stored_dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def load_required(self, name: str, role: str = "matrix", device="cpu") -> WeightHandle:
        require(name in self._where, f"missing required tensor: {name}")
        return self._load(name, role, device)

    def load_optional(self, name: str, role: str = "matrix", device="cpu") -> Optional[WeightHandle]:
        return self._load(name, role, device) if name in self._where else None

    def _load(self, name, role, device) -> WeightHandle:
        f = self._where[name]
        kept = _kept_dtype(f.dtype(name), role)
        require(kept is not None, f"tensor '{name}' is stored as {f.dtype(name)}, which cannot serve as a {role}")
        t = f.read(name)
        if t.dtype != kept:
            t = t.to(kept)
        if str(device) != "cpu":
            t = t.to(device, non_blocking=False)
        return WeightHandle(name, t.dtype, tuple(t.shape), t)

    def check(self, specs: Sequence[TensorSpec]) -> None:
        """Compare the folder with what the model expects; one error lists everything wrong."""
        expected = {s.name: s for s in specs}
        missing = [s.name for s in specs if not s.optional and s.name not in self._where]
        unexpected = sorted(n for n in self._where if n not in expected)
        wrong_shape, wrong_dtype = [], []
        for s in specs:
            if s.name not in self._where:
                continue
            got = self.stored_shape(s.name)
            if tuple(got) != tuple(s.shape):
                wrong_shape.append(f"{s.name}: got {list(got)}, expected {list(s.shape)}")
            if _kept_dtype(self.stored_dtype(s.name), s.role) is None:
                wrong_dtype.append(f"{s.name}: stored as {self.stored_dtype(s.name)}, needed as a {s.role}")
        if missing or unexpected or wrong_shape or wrong_dtype:
            lines = [f"weights in '{self.model_dir}' do not match the model:"]
            for title, items in (("missing tensors", missing), ("unexpected tensors", unexpected),
                                 ("wrong shapes", wrong_shape), ("wrong dtypes", wrong_dtype)):
                if items:
                    lines.append(f"  {title} ({len(items)}):")
                    lines.extend(f"    {i}" for i in items)
            raise CitlaliError("\n".join(lines))

    def load_all(self, specs: Sequence[TensorSpec], device="cpu", progress=None) -> Dict[str, WeightHandle]:
        self.check(specs)
        out: Dict[str, WeightHandle] = {}
        for i, s in enumerate(specs):
            if s.name in self._where:
                out[s.name] = self._load(s.name, s.role, device)
            if progress is not None:
                progress(i + 1, len(specs))
        return out

    def close(self):
        for f in self._files:
            f.close()
        self._files = []
        self._where = {}
