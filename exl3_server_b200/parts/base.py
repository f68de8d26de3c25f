"""What every part is built with and what it may ask of the cache.

Interfaces (duck-typed; the classes below only document them):

``Norm``           ``tensor_specs(spec, prefix)``; ``__init__(spec, tensors, prefix, ctx)``;
                   ``add_norm(stream, rows=None, out_scale=1.0) -> r``: folds the stream's
                   pending sublayer output into the float32 residual and returns the
                   normed rows in the activation dtype.
``Position``       ``__init__(spec, head_dim, ctx)``;
                   ``rotate_and_store(qkv, batch, kv, heads, kv_heads, head_dim)``: encodes
                   positions into q and k inside ``qkv`` and writes k, v to the cache view
                   (when the view owns its storage).
``Mixer``          ``tensor_specs(spec, prefix)``; ``__init__(spec, tensors, prefix, ctx)``;
                   ``cache_request() -> KVRequest | None``; ``state_request() -> StateRequest | None``;
                   ``forward(x, batch, kv, state) -> y`` with x, y ``[tokens, width]``.
``FeedForward``    ``tensor_specs(spec, prefix)``; ``__init__(spec, tensors, prefix, ctx)``;
                   ``forward(x, batch) -> y``.
``Arrangement``    ``__init__(layer_spec, mixer, feed_forward, mixer_norm, feed_forward_norm)``;
                   ``forward(stream, batch, kv, state)``.

``batch`` is an ``engine.batch.StepBatch``; ``kv`` a ``cache.kv.KVLayerView`` or None;
``state`` the layer's ``[slots, *shape]`` tensor or None (rows are picked with
``batch.slot_ids``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class BuildContext:
    dtype: torch.dtype            # activations and matrix weights: bfloat16 or float32
    device: torch.device


@dataclass(frozen=True)
class KVRequest:
    """Keys and values for every position (window 0) or the last ``window``.  ``value_dim`` is the width of a
    value per head when it differs from the key's (0: the same), as in mixers that keep narrow keys or a
    compressed value."""
    kv_heads: int
    head_dim: int
    window: int = 0
    value_dim: int = 0


@dataclass(frozen=True)
class StateRequest:
    """A tensor of fixed size per sequence, zero when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class ResidualStream:
    """The float32 residual ``h`` plus at most one sublayer output that has
    not been added yet.  The add is fused into the next norm."""

    def __init__(self, h: torch.Tensor):
        self.h = h
        self.pending: Optional[torch.Tensor] = None
        self.pending_scale: float = 1.0
        # (norm, RawNormed): what ``norm`` needs for its output over the residual as it stands, left by a
        # projection that folded its output into the residual in its own kernel (see NormAfter)
        self.normed = None

    def push(self, y: torch.Tensor, scale: float) -> None:
        if self.pending is not None:
            raise RuntimeError("residual stream already holds an output that was not folded in")
        self.pending = y
        self.pending_scale = scale
        self.normed = None

    def take_normed(self, norm):
        """What a projection has left for ``norm`` over the residual as it stands (a ``RawNormed``), or None."""
        got, self.normed = self.normed, None
        if got is not None and self.pending is None and got[0] is norm:
            return got[1]
        return None

    def take(self):
        y, s = self.pending, self.pending_scale
        self.pending, self.pending_scale = None, 1.0
        return y, s


class RawNormed:
    """A norm's output in two pieces, as a projection kernel left it: ``x_raw = h * weight`` (bfloat16) and the
    sums of squares of ``h`` per batch row and block of 16 features (``ss [16, blocks]``); the output itself is
    ``x_raw * rsqrt(ss.sum(1) / width + eps)`` per row.  A projection that takes it applies the factor to its
    results (``Linear`` does); anyone else calls ``materialize()``."""

    def __init__(self, x_raw: torch.Tensor, ss: torch.Tensor, eps: float, width: int):
        self.x_raw, self.ss, self.eps, self.width = x_raw, ss, eps, width

    @property
    def shape(self):
        return self.x_raw.shape

    def materialize(self, out_scale: float = 1.0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The norm's output, of all rows or of the rows listed (a prompt's last position, say)."""
        n = self.x_raw.shape[0]
        x_raw, ss = self.x_raw, self.ss[:n]
        if rows is not None:
            x_raw, ss = x_raw.index_select(0, rows.long()), ss.index_select(0, rows.long())
        inv = torch.rsqrt(ss.sum(dim=1) / float(self.width) + self.eps)
        return (x_raw.float() * (inv * out_scale)[:, None]).to(x_raw.dtype)


class NormAfter:
    """An offer to a part's last projection: instead of returning its output ``y`` to be added later, it may,
    where its kernel can, add ``y * scale`` to the residual ``stream.h`` itself and leave what ``norm`` needs
    for its output over the new residual in ``stream.normed`` (then ``done`` is set, the projection returns
    None and the caller adds nothing).  A part that takes the offer declares ``takes_then = True`` and passes
    ``then`` to its last ``Linear`` call; everything still works when the offer is ignored."""

    def __init__(self, stream: ResidualStream, scale: float, norm):
        self.stream = stream
        self.scale = scale
        self.norm = norm
        self.done = False
