"""Arrangements of a layer's parts.

``prenorm``: ``h += rho * mixer(norm1(h))`` then ``h += rho * ff(norm2(h))``
(src/model.cpp:556-586, with rho = 1 there).  The sublayer output is
multiplied by ``residual_scale`` and then added, in float32, inside the next
norm's kernel.
"""
from __future__ import annotations

from .base import ResidualStream
from .registry import register_arrangement
from .spec import LayerSpec


class PreNormBlock:
    def __init__(self, spec: LayerSpec, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, stream: ResidualStream, batch, kv, state) -> None:
        r = self.mixer_norm.add_norm(stream)
        stream.push(self.mixer.forward(r, batch, kv, state), self.spec.residual_scale)
        r = self.feed_forward_norm.add_norm(stream)
        stream.push(self.feed_forward.forward(r, batch), self.spec.residual_scale)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward, self.mixer_norm,
                                              self.feed_forward_norm) if hasattr(p, "weight_bytes"))


register_arrangement("prenorm", PreNormBlock)
