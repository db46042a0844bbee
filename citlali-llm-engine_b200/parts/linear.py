"""Dense linear maps: y = x . W^T with W stored [out, in] row-major, no bias.

The reference routes every projection through ``LinearBackend::forward(weight, input,
output)`` (include/citlali/model/linear_backend.h:10-21), which picks a kernel from the
weight's storage (src/model/linear_backend.cpp:17-68).  This is the same seam: model parts
call :class:`DenseLinear`; it picks the kernel from the compute dtype and the shape.

* float32: the CUDA-core product (k ascending, one chain per output element).
* bfloat16: the tensor-core product where its shape rules hold (inner size a multiple of 8,
  16-byte aligned rows), else the CUDA-core product on bfloat16 storage.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from ..errors import require
from ..weights.loader import TensorSpec


class DenseLinear:
    def __init__(self, names: Sequence[str], out_features: Sequence[int], in_features: int,
                 interleave_run: Optional[int] = None):
        """One matrix, or several with the same input stacked along the output axis (``names``
        in order).  ``interleave_run``: for exactly two stacked matrices, alternate runs of that
        many rows of the first and of the second (gate and up of a gated feed-forward)."""
        self.names = list(names)
        self.out_splits = list(out_features)
        self.in_features = in_features
        self.out_features = sum(out_features)
        self.interleave_run = interleave_run
        if interleave_run is not None:
            require(len(self.names) == 2 and out_features[0] == out_features[1]
                    and out_features[0] % interleave_run == 0,
                    "interleaving needs two matrices of equal height that the run divides")
        self.weight: Optional[torch.Tensor] = None
        self.error_flag = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(n, (o, self.in_features), "matrix") for n, o in zip(self.names, self.out_splits)]

    def bind(self, weights, ctx):
        """One device buffer for the stacked matrix; every named matrix is copied straight into its rows
        (alternating runs if interleaved), converted to the compute dtype on the way."""
        handles = [weights[n] for n in self.names]
        for n, h, o in zip(self.names, handles, self.out_splits):
            require(tuple(h.shape) == (o, self.in_features),
                    f"unexpected tensor shape for {n}: got {list(h.shape)}, expected {[o, self.in_features]}")
        w = torch.empty((self.out_features, self.in_features), dtype=ctx.dtype, device=ctx.device)
        if self.interleave_run is not None:
            r = self.interleave_run
            runs = w.view(-1, 2, r, self.in_features)          # [run index, gate or up, row in run, in]
            for k, h in enumerate(handles):
                h.copy_into(runs[:, k])
        else:
            at = 0
            for h, o in zip(handles, self.out_splits):
                h.copy_into(w[at:at + o])
                at += o
        self.weight = w
        self.dtype = ctx.dtype
        self.error_flag = ctx.error_flag

    # ---- a norm in front of this map, done by the map ----------------------------------------------------------
    def can_take_normed_rows(self) -> bool:
        """Bound in bfloat16 with shapes the tensor-core product takes: it can then read un-normalised rows and scale
        its result rows instead (:class:`~.base.NormedRows`), once the norm's gain is folded into its weights."""
        return (self.weight is not None and self.dtype == torch.bfloat16 and self.in_features % 32 == 0
                and (self.interleave_run is None or (self.interleave_run == 16 and self.out_features % 32 == 0)))

    def can_emit_normed_rows(self) -> bool:
        return self.weight is not None and self.dtype == torch.bfloat16 and self.in_features % 8 == 0 and self.out_features % 32 == 0

    def fold_input_gain(self, gain: torch.Tensor) -> None:
        """W[n, k] *= gain[k] (in 32-bit, rounded once): x . (g * W)^T = (x * g) . W^T, so the norm in front of this map
        no longer multiplies by its gain."""
        require(gain.numel() == self.in_features, "the gain's length is not the map's input size")
        w = self.weight
        for r0 in range(0, w.shape[0], 8192):            # in pieces: no second copy of a large matrix in 32-bit
            piece = w[r0:r0 + 8192]
            piece.copy_((piece.float() * gain.float().to(w.device)[None, :]).to(w.dtype))

    def bind_shared(self, weight: torch.Tensor, ctx):
        """Use a matrix another part already holds (a head tied to the embedding)."""
        require(tuple(weight.shape) == (self.out_features, self.in_features), "shared matrix has the wrong shape")
        self.weight = weight
        self.dtype = ctx.dtype
        self.error_flag = ctx.error_flag

    def uses_tensor_cores(self, x: torch.Tensor) -> bool:
        return (self.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and self.in_features % 8 == 0
                and x.is_contiguous() and x.data_ptr() % 16 == 0)

    def forward_gated(self, x: torch.Tensor, run: int, row_scale=None):
        """For two stacked matrices interleaved in runs of 16 (gate, up): ``silu(gate) * up`` straight
        from the product's epilogue, or ``None`` if this shape cannot (call :meth:`forward`).  ``row_scale``: see
        :meth:`forward`."""
        rows = x.shape[0]
        if rows == 0 or run != 16 or self.out_features % 32 != 0 or not self.uses_tensor_cores(x):
            require(row_scale is None, "this shape has no gate epilogue to scale rows in")
            return None
        act = torch.empty((rows, self.out_features // 2), dtype=torch.bfloat16, device=x.device)
        ops.gemm_tc(x, self.weight, act, error_flag=self.error_flag, swiglu=True, row_scale=row_scale)
        return act

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                accumulate_into: Optional[torch.Tensor] = None, row_scale=None, emit=None) -> torch.Tensor:
        """``accumulate_into`` (float32 [rows, out]) receives ``+= x . W^T`` and is returned;
        otherwise a new tensor of ``out_dtype`` (default: the compute dtype).  Few rows, tensor-core shapes only:
        ``row_scale`` (``NormedRows.scale`` of the rows ``x`` stands for) scales the result rows; ``emit`` (a pair of
        buffers, with ``accumulate_into``) receives the updated rows as bfloat16 and their sums of squares."""
        rows = x.shape[0]
        if accumulate_into is not None:
            y = accumulate_into
        else:
            y = torch.empty((rows, self.out_features), dtype=out_dtype or self.dtype, device=x.device)
        if rows == 0:
            return y
        if self.dtype == torch.bfloat16 and ops.gemm_tc_accepts(x, self.weight, y):
            ops.gemm_tc(x, self.weight, y, accumulate=accumulate_into is not None, error_flag=self.error_flag,
                        row_scale=row_scale, emit=emit)
        else:
            require(row_scale is None and emit is None, "only the tensor-core product does a norm's work in its epilogue")
            ops.gemm_simt(x, self.weight, y, accumulate=accumulate_into is not None)
        return y

    @property
    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()
