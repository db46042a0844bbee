"""Arrangements of a layer's parts around the residual stream.

``pre_norm_residual`` is the reference's layer (src/model/qwen_model.cpp:306-374):
x += mixer(norm(x)); x += feed_forward(norm(x)).  The residual stream is float32 and the two
sums are 32-bit additions.  Either half may be absent from the layer's parts (a layer with a
mixer only, or a feed-forward only).

For few rows in bfloat16 (decoding) the two norms need no kernels of their own: the product that ends a sub-layer also
writes the updated residual rows as bfloat16 with the sums of their squares, the product that begins the next sub-layer
reads those rows and scales its result by the inverse root mean square, and the norm's gain is multiplied into that
product's weights once, when the layer is bound (x . (g W)^T rsqrt(mean x^2 + eps) = (x rsqrt(...) g) . W^T).  That is
an arrangement between this block, RMSNorm and parts that say they can (``can_absorb_norm``); other parts and other
norms run the plain way.

A block is given the layer's description and builds its parts from the registries by the
names it knows; another arrangement (four norms a layer, one norm for a mixer and a
feed-forward side by side) is another class registered under another kind, with part names of
its own.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import NormedRows, build_part, register_part
from .norm import RMSNorm

_FEW_ROWS = 128        # up to here the product always runs the form whose epilogue can do a norm's work


class PreNormResidualBlock:
    def __init__(self, layer_spec):
        has = layer_spec.parts.__contains__
        self.mixer = self.mixer_norm = self.feed_forward = self.feed_forward_norm = None
        if has("mixer"):
            self.mixer_norm = build_part("norm", layer_spec.part("mixer_norm"))
            self.mixer = build_part("mixer", layer_spec.part("mixer"))
        if has("feed_forward"):
            self.feed_forward_norm = build_part("norm", layer_spec.part("feed_forward_norm"))
            self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward"))

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        return [t for p in self.parts() for t in p.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement() if self.mixer is not None else None

    def bind(self, weights, ctx):
        for p in self.parts():
            p.bind(weights, ctx)
        self.norms_in_products = (
            self.mixer is not None and self.feed_forward is not None and ctx.dtype == torch.bfloat16
            and type(self.mixer_norm) is RMSNorm and type(self.feed_forward_norm) is RMSNorm
            and not self.mixer_norm.gain_downstream and not self.feed_forward_norm.gain_downstream
            and self.mixer_norm.size % 32 == 0 and self.mixer_norm.size == self.feed_forward_norm.size
            and callable(getattr(self.mixer, "can_absorb_norm", None)) and self.mixer.can_absorb_norm()
            and callable(getattr(self.feed_forward, "can_absorb_norm", None)) and self.feed_forward.can_absorb_norm())
        if self.norms_in_products:
            self.mixer.fold_norm_gain(self.mixer_norm.gain_moves_downstream())
            self.feed_forward.fold_norm_gain(self.feed_forward_norm.gain_moves_downstream())

    def forward(self, x, batch, cache_view, write_cache=True):
        if getattr(self, "norms_in_products", False) and 0 < batch.rows <= _FEW_ROWS:
            return self._forward_norms_in_products(x, batch, cache_view, write_cache)
        if self.mixer is not None:
            self.mixer.forward(self.mixer_norm.forward(x), batch, cache_view, x, write_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(self.feed_forward_norm.forward(x), batch, x)
        return x

    def _forward_norms_in_products(self, x, batch, cache_view, write_cache):
        rows, hidden = x.shape
        def buffers():
            return (torch.empty((rows, hidden), dtype=torch.bfloat16, device=x.device),
                    torch.empty((rows, hidden // 32), dtype=torch.float32, device=x.device))
        carried = batch.norm_carry_in
        if carried is None or carried.rows.shape != (rows, hidden):
            rows_bf16, sumsq = buffers()                   # the rows came from somewhere that emitted nothing
            ops.norm_inputs(x, rows_bf16, sumsq)
            carried = NormedRows(rows_bf16, sumsq, hidden)
        after_mixer = buffers()
        self.mixer.forward(carried.with_eps(self.mixer_norm.eps), batch, cache_view, x, write_cache, emit=after_mixer)
        after_ff = buffers()
        self.feed_forward.forward(NormedRows(after_mixer[0], after_mixer[1], hidden, self.feed_forward_norm.eps), batch, x,
                                  emit=after_ff)
        batch.norm_carry = NormedRows(after_ff[0], after_ff[1], hidden)
        return x


register_part("block", "pre_norm_residual", PreNormResidualBlock)
