"""Causal grouped-query attention over the cache, with optional per-head q/k RMSNorm.

The order of operations is the reference's (src/model/qwen_model.cpp:315-351): q, k, v
projections without bias; RMSNorm over each q and k head with a gain [head_dim] shared by all
heads and the layer norms' eps, before the rotation; v untouched; k and v stored at the
token's position; query head j reads KV head j // (heads / kv_heads); scores scaled by
1/sqrt(head_dim); keys 0..p for the token at position p (no window in the reference; a
window is a parameter here); softmax and value sum in 32-bit; output projection added to the
residual stream.

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (None: no head norm),
position ({"kind": ..., ...}), window (None: all keys), kv_projection (False: the layer has no
k/v matrices and only reads another layer's cache).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..cache import KVRequirement
from ..errors import require
from ..weights.loader import TensorSpec
from .base import NormedRows, bind_gain, part_class, register_part
from .linear import DenseLinear


class GQAttention:
    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.nq = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        self.eps = params.get("qk_norm_eps")
        self.window = params.get("window")
        self.kv_projection = bool(params.get("kv_projection", True))
        require(self.nq % self.nkv == 0,
                f"{prefix}: {self.nq} query heads are not a multiple of {self.nkv} key/value heads")
        require(self.d % 2 == 0, f"{prefix}: head size {self.d} must be even")
        require(self.window is None or int(self.window) > 0, f"{prefix}: window must be positive or None")
        pos = dict(params.get("position") or {"kind": "none"})
        self.position = part_class("position", pos.pop("kind"))(pos, self.d)
        self.prefix = prefix
        names = [f"{prefix}.q_proj.weight"]
        outs = [self.nq * self.d]
        if self.kv_projection:
            names += [f"{prefix}.k_proj.weight", f"{prefix}.v_proj.weight"]
            outs += [self.nkv * self.d, self.nkv * self.d]
        self.qkv = DenseLinear(names, outs, self.hidden)
        self.o = DenseLinear([f"{prefix}.o_proj.weight"], [self.hidden], self.nq * self.d)
        self.q_gain = self.k_gain = None

    @property
    def graph_safe(self) -> bool:
        """A step of single tokens reads slots and positions from device memory only: true once bound
        to a dtype and head size that the split-context kernel takes; the other attention kernels size
        their launch from the host's lists."""
        if getattr(self, "dtype", None) is None or not ops.attention_steps_from_device(self.dtype, self.d):
            return False
        return self.position.inv_freq is not None or bool(getattr(self.position, "graph_safe", False))

    # ---- what it needs ---------------------------------------------------------------
    def tensor_specs(self):
        specs = self.qkv.tensor_specs() + self.o.tensor_specs()
        if self.eps is not None:
            specs.append(TensorSpec(f"{self.prefix}.q_norm.weight", (self.d,), "gain"))
            if self.kv_projection:
                specs.append(TensorSpec(f"{self.prefix}.k_norm.weight", (self.d,), "gain"))
        return specs

    def cache_requirement(self):
        if not self.kv_projection:
            return None
        return KVRequirement(self.nkv, self.d, None if self.window is None else int(self.window))

    def bind(self, weights, ctx):
        self.qkv.bind(weights, ctx)
        self.o.bind(weights, ctx)
        if self.eps is not None:
            self.q_gain = bind_gain(weights, f"{self.prefix}.q_norm.weight", self.d, ctx)
            self.k_gain = (bind_gain(weights, f"{self.prefix}.k_norm.weight", self.d, ctx)
                           if self.kv_projection else self.q_gain)
            if self.k_gain.dtype != self.q_gain.dtype:
                self.k_gain = self.k_gain.to(torch.float32)
                self.q_gain = self.q_gain.to(torch.float32)
        self.fused_position = self.position.inv_freq is not None
        if self.fused_position:
            self.rotary_dim = int(self.position.rotary_dim)
            self.inv_freq = self.position.inv_freq.to(ctx.device)
        else:
            require(callable(getattr(self.position, "apply", None)),
                    f"{self.prefix}: a position encoding gives either inv_freq or apply()")
            self.rotary_dim = self.d
            self.inv_freq = torch.zeros(self.d // 2, dtype=torch.float32, device=ctx.device)   # no rotation by the kernel
        self.dtype = ctx.dtype

    # ---- the norm in front of this part, done by its products ---------------------------------------------------
    def can_absorb_norm(self) -> bool:
        return self.qkv.can_take_normed_rows() and self.o.can_emit_normed_rows()

    def fold_norm_gain(self, gain: torch.Tensor) -> None:
        self.qkv.fold_input_gain(gain)

    # ---- one step ----------------------------------------------------------------------
    def forward(self, h, batch, cache_view, residual, write_cache=True, emit=None):
        """``h``: the normed rows, or :class:`~.base.NormedRows` (few rows; after :meth:`fold_norm_gain`).  ``emit``: a pair
        of buffers that the output projection fills with what the next norm needs of the updated residual rows."""
        require(cache_view is not None, f"{self.prefix}: attention needs a key/value cache")
        req = cache_view.requirement
        nkv_here = self.nkv if self.kv_projection else 0
        require(req.head_dim == self.d and req.num_kv_heads == self.nkv,
                f"{self.prefix}: the cache holds {req.num_kv_heads} heads of {req.head_dim}, "
                f"the layer has {self.nkv} of {self.d}")
        if isinstance(h, NormedRows):
            qkv = self.qkv.forward(h.rows, row_scale=h.scale)
        else:
            qkv = self.qkv.forward(h)
        store = write_cache and self.kv_projection
        common = (batch.row_slot, batch.row_pos, cache_view.page_table, cache_view.keys, cache_view.values,
                  cache_view.page_size, self.nq, nkv_here, self.d, float(self.eps or 0.0))
        if self.fused_position:
            ops.qk_norm_rope_cache(qkv, self.q_gain, self.k_gain, self.inv_freq, self.rotary_dim, *common,
                                   write_cache=store)
        else:
            # head norm with the keys kept in the row, the encoding's own work on q and k, then the store
            ops.qk_norm_rope_cache(qkv, self.q_gain, self.k_gain, self.inv_freq, self.rotary_dim, *common,
                                   write_cache="keys_in_place" if store else False)
            self.position.apply(qkv, batch, self.nq, nkv_here, self.d)
            if store:
                ops.qk_norm_rope_cache(qkv, None, None, self.inv_freq, self.rotary_dim, *common, write_cache=True)
        out = torch.empty((batch.rows, self.nq * self.d), dtype=self.dtype, device=qkv.device)
        ops.attention(qkv, qkv.shape[1], cache_view, batch, out, self.nq, self.nkv, self.d,
                      int(self.window or 0), 1.0 / math.sqrt(self.d))
        self.o.forward(out, accumulate_into=residual, emit=emit)
        return residual


register_part("mixer", "gqa_attention", GQAttention)
