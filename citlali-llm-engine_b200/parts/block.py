"""Arrangements of a layer's parts around the residual stream.

``pre_norm_residual`` is the reference's layer (src/model/qwen_model.cpp:306-374):
x += mixer(norm(x)); x += feed_forward(norm(x)).  The residual stream is float32 and the two
sums are 32-bit additions.  Either half may be absent from the layer's parts (a layer with a
mixer only, or a feed-forward only).

A block is given the layer's description and builds its parts from the registries by the
names it knows; another arrangement (four norms a layer, one norm for a mixer and a
feed-forward side by side) is another class registered under another kind, with part names of
its own.
"""
from __future__ import annotations

from .base import build_part, register_part


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

    def forward(self, x, batch, cache_view, write_cache=True):
        if self.mixer is not None:
            self.mixer.forward(self.mixer_norm.forward(x), batch, cache_view, x, write_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(self.feed_forward_norm.forward(x), batch, x)
        return x


register_part("block", "pre_norm_residual", PreNormResidualBlock)
