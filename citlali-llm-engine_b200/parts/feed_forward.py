"""The gated feed-forward: act = silu(W_gate h) * (W_up h), y = W_down act, added to the
residual stream (src/model/qwen_model.cpp:360-374; the gate is swiglu_kernel,
src/compute/cuda/kernels.cu:474-482).  The reference runs gate and up as two products; here
their matrices are stacked with rows alternating in runs, so that one product yields both
and matching gate and up values lie next to each other for the gate kernel.

Parameters: hidden_size, intermediate_size.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import NormedRows, register_part
from .linear import DenseLinear

_RUN = 16


class GatedSiluFeedForward:
    graph_safe = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.run = _RUN if self.inter % _RUN == 0 else self.inter
        self.gate_up = DenseLinear([f"{prefix}.gate_proj.weight", f"{prefix}.up_proj.weight"],
                                   [self.inter, self.inter], self.hidden, interleave_run=self.run)
        self.down = DenseLinear([f"{prefix}.down_proj.weight"], [self.hidden], self.inter)

    def tensor_specs(self):
        return self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, weights, ctx):
        self.gate_up.bind(weights, ctx)
        self.down.bind(weights, ctx)
        self.dtype = ctx.dtype

    def can_absorb_norm(self) -> bool:
        return self.run == _RUN and self.gate_up.can_take_normed_rows() and self.down.can_emit_normed_rows()

    def fold_norm_gain(self, gain: torch.Tensor) -> None:
        self.gate_up.fold_input_gain(gain)

    def forward(self, h, batch, residual, emit=None):
        """``h``: the normed rows, or :class:`~.base.NormedRows` (few rows; after :meth:`fold_norm_gain`).  ``emit``: a pair
        of buffers that the down projection fills with what the next norm needs of the updated residual rows."""
        if isinstance(h, NormedRows):
            act = self.gate_up.forward_gated(h.rows, self.run, row_scale=h.scale)
        else:
            act = self.gate_up.forward_gated(h, self.run)          # gate in the product's epilogue
            if act is None:
                act = torch.empty((h.shape[0], self.inter), dtype=self.dtype, device=h.device)
                ops.swiglu(self.gate_up.forward(h), act, self.run)
        self.down.forward(act, accumulate_into=residual, emit=emit)
        return residual


register_part("feed_forward", "gated_silu", GatedSiluFeedForward)
