"""Arrangements of a layer's parts around the residual stream.

``pre_norm_residual`` is the reference's layer (src/model/qwen_model.cpp:306-374):
x += mixer(norm(x)); x += feed_forward(norm(x)).  The residual stream is float32 and the two
sums are 32-bit additions.
"""
from __future__ import annotations

from .base import part_class, register_part


class PreNormResidualBlock:
    def __init__(self, layer_spec):
        s = layer_spec
        self.mixer_norm = part_class("norm", s.mixer_norm.kind)(s.mixer_norm.params, s.mixer_norm.prefix)
        self.mixer = part_class("mixer", s.mixer.kind)(s.mixer.params, s.mixer.prefix)
        self.feed_forward_norm = part_class("norm", s.feed_forward_norm.kind)(
            s.feed_forward_norm.params, s.feed_forward_norm.prefix)
        self.feed_forward = part_class("feed_forward", s.feed_forward.kind)(
            s.feed_forward.params, s.feed_forward.prefix)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def tensor_specs(self):
        return [t for p in self.parts() for t in p.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def bind(self, weights, ctx):
        for p in self.parts():
            p.bind(weights, ctx)

    def forward(self, x, batch, cache_view, write_cache=True):
        self.mixer.forward(self.mixer_norm.forward(x), batch, cache_view, x, write_cache)
        self.feed_forward.forward(self.feed_forward_norm.forward(x), batch, x)
        return x


register_part("block", "pre_norm_residual", PreNormResidualBlock)
