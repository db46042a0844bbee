"""RMSNorm over the hidden size: y = x * rsqrt(mean(x^2) + eps) * gain, eps inside the root,
the gain multiplies (no 1 + gain) -- rms_norm_kernel, src/compute/cuda/kernels.cu:73-92.
Input is the float32 residual stream; the sum of squares, the root and the product are
32-bit, rounded once at the store to the compute dtype."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import require
from ..weights.loader import TensorSpec
from .base import register_part


class RMSNorm:
    graph_safe = True

    def __init__(self, params, prefix: str):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = f"{prefix}.weight"
        self.gain = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), "gain")]

    def bind(self, weights, ctx):
        g = weights[self.name].tensor
        require(tuple(g.shape) == (self.size,),
                f"unexpected tensor shape for {self.name}: got {list(g.shape)}, expected {[self.size]}")
        # a gain stored in 32-bit stays 32-bit; the 32-bit path widens a bfloat16 gain (exact)
        self.gain = g.to(device=ctx.device, dtype=torch.float32 if ctx.is_float32 else g.dtype).contiguous()
        self.dtype = ctx.dtype

    def forward(self, x: torch.Tensor, row_index=None) -> torch.Tensor:
        rows = x.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.size), dtype=self.dtype, device=x.device)
        ops.rms_norm(x, self.gain, self.eps, out, row_index)
        return out


register_part("norm", "rms_norm", RMSNorm)
