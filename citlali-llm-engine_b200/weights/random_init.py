"""Random weights from a configuration and a seed.

The reference has no such mode; it exists here so that tests and benchmarks need no
checkpoint.  Every tensor's values depend only on ``(seed, tensor name)``: linear and
embedding matrices are N(0, matrix_std), norm gains are 1 + N(0, gain_spread).  The
generator runs on the host for model folders, so that every reader of the folder sees
the same bits; the device variant serves benchmarks, where nothing is compared.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Sequence

import torch

from ..errors import require
from .loader import SINGLE_FILE, TensorSpec
from .safetensors_io import write_safetensors

_FNV_OFFSET = 0xCBF29CE484222325
_FNV_PRIME = 0x100000001B3


def name_seed(seed: int, name: str) -> int:
    """64-bit FNV-1a of the tensor name, mixed with the seed."""
    h = _FNV_OFFSET ^ (seed & 0xFFFFFFFFFFFFFFFF)
    for b in name.encode("utf-8"):
        h = ((h ^ b) * _FNV_PRIME) & 0xFFFFFFFFFFFFFFFF
    return h & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu",
                  matrix_std: float = 0.02, gain_spread: float = 0.1) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(name_seed(seed, spec.name))
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.role == "gain":
        t = t.mul_(gain_spread).add_(1.0)
    else:
        t = t.mul_(matrix_std)
    return t.to(dtype)


def random_weights(specs: Sequence[TensorSpec], seed: int, dtype: torch.dtype, device="cpu",
                   matrix_std: float = 0.02, gain_spread: float = 0.1) -> Dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, dtype, device, matrix_std, gain_spread) for s in specs}


def write_random_model(model_dir: str, config, seed: int, dtype="bfloat16",
                       matrix_std: float = 0.02, gain_spread: float = 0.1) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (an architecture's typed
    configuration) into ``model_dir``.  Tied models store no head tensor."""
    from ..engine.model import expected_tensors   # describes tensors without touching a device
    torch_dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                   "float32": torch.float32, "fp32": torch.float32}.get(str(dtype).replace("torch.", ""))
    require(torch_dtype is not None, f"random weights can be written as bfloat16 or float32, not {dtype}")
    os.makedirs(model_dir, exist_ok=True)
    spec = config.to_model_spec()
    specs = [s for s in expected_tensors(spec) if not s.optional]
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(
        os.path.join(model_dir, SINGLE_FILE),
        lambda: ((s.name, random_tensor(s, seed, torch_dtype, "cpu", matrix_std, gain_spread)) for s in specs),
        metadata={"format": "pt", "random_seed": str(seed)})
    return model_dir
