"""Binding tensors by name: ``WeightLoader`` reads a model folder, ``WeightHandle`` is what
model code sees.

The reference's loader finds a tensor by its GGUF name, converts it and uploads it
(include/citlali/model/weight_loader.h:20-61, src/model/weight_loader.cpp:377-467) and the
model checks every shape at load (src/model/qwen_model.cpp:29-34, :156-173), failing on the
first problem.  Here the names are the checkpoint's own (HF) names, the stored dtype is
kept (bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 stays float16 until
a part converts it: exactly for the 32-bit path, rounded once for the bfloat16 path; integer
tables become int32), and all problems of a folder are reported together in one error.

Nothing is read when a handle is made.  A part either asks for ``handle.tensor`` (a host copy, for
small things such as gains) or gives the handle the device buffer the values belong in
(``handle.copy_into(dst)``): the loader then streams the tensor from the memory map through two
pinned staging buffers into ``dst``, piece by piece, converting to ``dst``'s dtype on the device.
The checkpoint is never held in host memory as a whole, and a stacked or interleaved matrix is
filled in place with no second device copy.
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


class WeightHandle:
    """A tensor of the checkpoint as model code sees it: name, dtype and shape at once, the values on
    demand.  ``tensor`` gives a host (or, for generated weights, device) tensor in the handle's dtype;
    ``copy_into(dst)`` fills ``dst`` (any device, any floating dtype, same number of elements, possibly a
    strided view) with the values."""

    def __init__(self, name: str, dtype: torch.dtype, shape: Tuple[int, ...], tensor: Optional[torch.Tensor] = None,
                 produce=None, stream=None):
        self.name = name
        self.dtype = dtype
        self.shape = tuple(shape)
        self._tensor = tensor
        self._produce = produce        # () -> tensor, called at every access: nothing is kept
        self._stream = stream          # (dst) -> None

    @property
    def tensor(self) -> torch.Tensor:
        if self._tensor is not None:
            return self._tensor
        require(self._produce is not None, f"tensor '{self.name}' has no values behind its handle")
        return self._produce()

    def copy_into(self, dst: torch.Tensor) -> None:
        n = 1
        for d in self.shape:
            n *= d
        require(dst.numel() == n, f"tensor '{self.name}' has {n} elements, its destination {dst.numel()}")
        if self._stream is not None:
            self._stream(dst)
        else:
            t = self.tensor
            dst.copy_(t.reshape(dst.shape))

    @property
    def out_features(self) -> int:      # rows of an [out, in] matrix (weight_loader.h:29-32)
        return self.shape[0]

    @property
    def in_features(self) -> int:
        return self.shape[1]

    @property
    def nbytes(self) -> int:
        n = torch.tensor([], dtype=self.dtype).element_size()
        for d in self.shape:
            n *= d
        return n


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def _kept_dtype(stored: torch.dtype, role: str) -> Optional[torch.dtype]:
    """The dtype a stored tensor is kept in; ``None`` if the stored dtype cannot serve the role."""
    if role == "table":
        return torch.int32 if stored in _INTS else None
    if stored in (torch.float32, torch.float64):
        return torch.float32
    if stored in (torch.bfloat16, torch.float16):
        return stored
    return None


STAGE_BYTES = 64 << 20      # one piece of a streamed tensor; two such pinned buffers exist while a model loads


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
        """A handle that reads when asked.  ``device`` other than the CPU: ``tensor`` arrives there."""
        f = self._where[name]
        kept = _kept_dtype(f.dtype(name), role)
        require(kept is not None, f"tensor '{name}' is stored as {f.dtype(name)}, which cannot serve as a {role}")

        def produce():
            t = f.read(name)
            if t.dtype != kept:
                t = t.to(kept)
            return t if str(device) == "cpu" else t.to(device, non_blocking=False)

        return WeightHandle(name, kept, f.shape(name), produce=produce, stream=lambda dst: self._stream(f, name, dst))

    # ---- streaming ----------------------------------------------------------------------
    def _stage(self, nbytes: int):
        """One of two pinned buffers, after the copy that last left it has finished."""
        if not hasattr(self, "_stages"):
            self._stages, self._stage_events, self._stage_at = [None, None], [None, None], 0
        i = self._stage_at = 1 - self._stage_at
        if self._stage_events[i] is not None:
            self._stage_events[i].synchronize()
        if self._stages[i] is None or self._stages[i].numel() < nbytes:
            self._stages[i] = torch.empty(max(nbytes, STAGE_BYTES), dtype=torch.uint8, pin_memory=True)
        return i, self._stages[i]

    def _stream(self, f: SafetensorsFile, name: str, dst: torch.Tensor) -> None:
        src = f.view(name)                              # over the memory map: nothing is read yet
        if src.numel() == 0:
            return
        src = src.reshape(dst.shape) if dst.dim() > 0 else src.reshape(())
        if dst.device.type != "cuda" or dst.dim() == 0:
            dst.copy_(src)
            return
        item = src.element_size()
        row_bytes = (src.numel() // src.shape[0]) * item
        rows_per_piece = max(1, STAGE_BYTES // max(row_bytes, 1))
        for r0 in range(0, src.shape[0], rows_per_piece):
            piece = src[r0:r0 + rows_per_piece]
            i, stage = self._stage(piece.numel() * item)
            host = stage[:piece.numel() * item].view(src.dtype).view(piece.shape)
            host.copy_(piece)                           # file pages -> pinned memory
            target = dst[r0:r0 + rows_per_piece]
            if target.dtype == host.dtype and target.is_contiguous():
                target.copy_(host, non_blocking=True)
            else:                                       # the dtype changes, or the rows interleave with another tensor's
                target.copy_(host.to(dst.device, non_blocking=True))
            if self._stage_events[i] is None:
                self._stage_events[i] = torch.cuda.Event()
            self._stage_events[i].record(torch.cuda.current_stream(dst.device))

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
        """Handles for every expected tensor the folder has, after :meth:`check`.  They read when a part
        asks (see the module's head); ``progress(done, total)`` is called as handles are made."""
        self.check(specs)
        out: Dict[str, WeightHandle] = {}
        for i, s in enumerate(specs):
            if s.name in self._where:
                out[s.name] = self._load(s.name, s.role, device)
            if progress is not None:
                progress(i + 1, len(specs))
        return out

    def close(self):
        """Waits for copies in flight, then lets go of the files and the staging buffers."""
        for ev in getattr(self, "_stage_events", []):
            if ev is not None:
                ev.synchronize()
        self._stages, self._stage_events = [None, None], [None, None]
        for f in self._files:
            f.close()
        self._files = []
        self._where = {}
