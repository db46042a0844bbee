"""Rotary position encoding, half-split pairing.

Reference: rope_kernel (src/compute/cuda/kernels.cu:485-521): for i in [0, d/2),
f_i = powf(theta, -2i/d), angle = float(position) * f_i, and the pair (x_i, x_{i+d/2}) is
rotated by that angle; the whole head is rotated and the position is the absolute index.
The reference evaluates powf on the device for every call; here f_i is tabulated once on the
host (in double, rounded to float32, which is what a correctly rounded powf returns) and the
kernels form the angle as the same float32 product and take sincosf of it.

Interface of a position encoding: ``__init__(params, head_dim)`` and ``rotary_dim``.  Either
``inv_freq`` (float32 ``[rotary_dim/2]`` on the host): the fused norm-rotate-cache kernel rotates the
first ``rotary_dim`` elements of every q and k head in pairs (i, i + rotary_dim/2) by
``position * inv_freq[i]`` and leaves the rest of the head as it is (``rotary_dim`` below the
head size: a partial rotation; zero frequencies: none).  Or ``inv_freq = None`` and
``apply(qkv, batch, num_q_heads, num_kv_heads, head_dim)``, which changes the q and k heads of the
projection's rows ``[rows, (q + 2 kv heads) * head_dim]`` in place, after their head norm and before the
keys are stored; ``batch.row_pos`` holds each row's position.  An encoding with ``apply`` says
``graph_safe = True`` only if it reads positions from the device tensors alone.
"""
from __future__ import annotations

import torch

from ..errors import require
from .base import register_part


class RotaryHalfSplit:
    def __init__(self, params, head_dim: int):
        self.theta = float(params["theta"])
        self.rotary_dim = int(params.get("rotary_dim", head_dim))
        require(self.theta > 0, f"rotary theta must be positive, got {self.theta}")
        require(self.rotary_dim % 2 == 0 and 0 < self.rotary_dim <= head_dim,
                f"rotary_dim {self.rotary_dim} must be even and at most the head size {head_dim}")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                  -2.0 * i / self.rotary_dim).to(torch.float32)


class NoPosition:
    """No rotation: a zero frequency table makes every angle zero."""

    def __init__(self, params, head_dim: int):
        self.rotary_dim = head_dim
        self.inv_freq = torch.zeros(head_dim // 2, dtype=torch.float32)


register_part("position", "rotary_half_split", RotaryHalfSplit)
register_part("position", "none", NoPosition)
