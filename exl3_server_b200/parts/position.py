"""Position encodings applied to queries and keys.

``rope``: half-split rotary embedding over the first ``dims`` features of each
head: for d < dims/2, ``f_d = theta^(-2d/dims)``, angle ``a = pos * scale * f_d``,
``x'[d] = x[d] cos a - x[d + dims/2] sin a``,
``x'[d + dims/2] = x[d + dims/2] cos a + x[d] sin a`` — the reference's
``mx::fast::rope(x, hd, traditional=false, theta, 1.0, offset)``
(src/model.cpp:566-567).  The frequency table (times ``scale``) is computed once in float64
and kept as two float32 rows, the rounded frequencies and what the rounding lost
(``kernels.rotary_table``): the kernels' float32 angles then stay right at large positions,
where ``pos * f`` with a rounded ``f`` is off by ``pos * 6e-8`` radians.  A scaled or extended
variant only needs another table.

``none``: no rotation; keys and values are still written to the cache.

A position part has ``rotate_and_store(qkv, batch, kv, heads, kv_heads, head_dim)``; it may also offer
``fused_rotation(head_dim)`` (see below), which lets the decode attention kernel do both jobs itself.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import BuildContext
from .registry import register_position
from .spec import PositionSpec


class RotaryPosition:
    def __init__(self, spec: PositionSpec, head_dim: int, ctx: BuildContext):
        if spec.dims % 2 != 0 or not 0 <= spec.dims <= head_dim:
            raise ValueError(f"rope: dims {spec.dims} must be even and at most head_dim {head_dim}")
        self.spec = spec
        self.inv_freq = K.rotary_table(self.frequencies(spec) * float(spec.scale)).to(ctx.device)

    @staticmethod
    def frequencies(spec: PositionSpec) -> torch.Tensor:
        """float64 ``theta^(-2d/dims)`` for d < dims / 2."""
        d = torch.arange(0, spec.dims // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * d / max(1, spec.dims))

    def rotate_and_store(self, qkv: torch.Tensor, batch, kv, heads: int, kv_heads: int, head_dim: int) -> None:
        write = kv is not None and kv.owns
        K.rope_kv_write(qkv, self.inv_freq, self.spec.dims, 1.0, batch.tok_pos,
                        batch.tok_seq, kv.block_table, kv.k if write else None, kv.v if write else None,
                        heads, kv_heads, head_dim, kv.page_size, write)


    def fused_rotation(self, head_dim: int):
        """``(frequency table, dims, position scale)`` when an attention kernel can apply this encoding itself (all of a head's
        features rotated, or none), else None: then ``rotate_and_store`` runs as a step of its own."""
        if self.spec.dims == 0:
            return None, 0, 1.0
        if self.spec.dims == head_dim:
            return self.inv_freq, self.spec.dims, 1.0                # the scale is in the table
        return None


class NoPosition(RotaryPosition):
    def __init__(self, spec: PositionSpec, head_dim: int, ctx: BuildContext):
        super().__init__(PositionSpec(kind="none", dims=0), head_dim, ctx)


register_position("rope", RotaryPosition)
register_position("none", NoPosition)
