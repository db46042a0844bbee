"""RMSNorm over the hidden size: y = x * rsqrt(mean(x^2) + eps) * gain, eps inside the root,
the gain multiplies (no 1 + gain) -- rms_norm_kernel, src/compute/cuda/kernels.cu:73-92.
Input is the float32 residual stream; the sum of squares, the root and the product are
32-bit, rounded once at the store to the compute dtype."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import bind_gain, register_part


class RMSNorm:
    graph_safe = True

    def __init__(self, params, prefix: str):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = f"{prefix}.weight"
        self.gain = None
        self.gain_downstream = False

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), "gain")]

    def bind(self, weights, ctx):
        self.gain = bind_gain(weights, self.name, self.size, ctx)
        self.dtype = ctx.dtype

    def gain_moves_downstream(self) -> torch.Tensor:
        """The part behind this norm has multiplied its weights by the gain: from now on the norm only divides by the
        root mean square (its kernel gets a gain of ones).  Returns the gain."""
        gain = self.gain
        self.gain = torch.ones_like(gain)
        self.gain_downstream = True
        return gain

    def forward(self, x: torch.Tensor, row_index=None) -> torch.Tensor:
        rows = x.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.size), dtype=self.dtype, device=x.device)
        ops.rms_norm(x, self.gain, self.eps, out, row_index)
        return out


register_part("norm", "rms_norm", RMSNorm)
