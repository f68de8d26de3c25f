"""Arrangements of a layer's parts.

``prenorm``: ``h += rho * mixer(norm1(h))`` then ``h += rho * ff(norm2(h))``
(src/model.cpp:556-586, with rho = 1 there).  The sublayer output is
multiplied by ``residual_scale`` and then added, in float32, inside the next
norm's kernel.
"""
from __future__ import annotations

from .base import NormAfter, ResidualStream
from .registry import register_arrangement
from .spec import LayerSpec


class PreNormBlock:
    def __init__(self, spec: LayerSpec, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    takes_after = True

    def forward(self, stream: ResidualStream, batch, kv, state, after=None) -> None:
        """``after``: the norm that the next block will apply first, if the caller knows it: the feed-forward's
        last projection may then apply it in its own kernel, as the mixer's may apply this block's second norm."""
        r = self._norm(self.mixer_norm, stream, self.mixer)
        self._run(self.mixer, (r, batch, kv, state), stream, self.feed_forward_norm)
        r = self._norm(self.feed_forward_norm, stream, self.feed_forward)
        self._run(self.feed_forward, (r, batch), stream, after)

    @staticmethod
    def _norm(norm, stream: ResidualStream, part):
        # a part whose first projection takes a norm's output in two pieces gets it that way when it is there
        if getattr(norm, "offers_raw", False) and getattr(part, "takes_raw", False):
            return norm.add_norm(stream, raw_ok=True)
        return norm.add_norm(stream)

    def _run(self, part, args, stream: ResidualStream, norm) -> None:
        then = None
        if norm is not None and getattr(part, "takes_then", False):
            then = NormAfter(stream, self.spec.residual_scale, norm)
            y = part.forward(*args, then=then)
        else:
            y = part.forward(*args)
        if then is None or not then.done:
            stream.push(y, self.spec.residual_scale)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward, self.mixer_norm,
                                              self.feed_forward_norm) if hasattr(p, "weight_bytes"))


register_arrangement("prenorm", PreNormBlock)
