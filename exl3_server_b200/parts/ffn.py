"""The dense gated feed-forward: ``y = (silu(r Wg^T) * (r Wu^T)) Wd^T``
(src/model.cpp:583-586; the reference applies SiLU unconditionally).  Gate and
up projections are one fused matrix; the product ``silu(g) * u`` is float32
inside its kernel.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext
from .linear import Linear
from .registry import register_feed_forward
from .spec import FeedForwardSpec


class SwiGLU:
    @staticmethod
    def tensor_specs(spec: FeedForwardSpec, prefix: str) -> List[TensorSpec]:
        out = [
            TensorSpec(prefix + "gate_proj.weight", (spec.inner, spec.width)),
            TensorSpec(prefix + "up_proj.weight", (spec.inner, spec.width)),
            TensorSpec(prefix + "down_proj.weight", (spec.width, spec.inner)),
        ]
        for name, n in (("gate_proj", spec.inner), ("up_proj", spec.inner), ("down_proj", spec.width)):
            out.append(TensorSpec(prefix + name + ".bias", (n,), optional=True, init="zeros"))
        return out

    def __init__(self, spec: FeedForwardSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        wg = tensors[prefix + "gate_proj.weight"].to(ctx.dtype)
        wu = tensors[prefix + "up_proj.weight"].to(ctx.dtype)
        bg, bu = tensors.get(prefix + "gate_proj.bias"), tensors.get(prefix + "up_proj.bias")
        z = torch.zeros(spec.inner, dtype=ctx.dtype, device=wg.device)
        has_bias = bg is not None or bu is not None
        bg = bg.to(ctx.dtype) if bg is not None else z
        bu = bu.to(ctx.dtype) if bu is not None else z
        # Rows in eights: eight gate rows, then the eight up rows of the same
        # features.  A 16-row tile of the decode projection then holds both halves
        # of eight features and applies silu(gate) * up before it writes.
        self.interleave = 8 if spec.inner % 8 == 0 else 0
        if self.interleave:
            n = spec.inner // 8
            w = torch.stack([wg.view(n, 8, -1), wu.view(n, 8, -1)], dim=1).reshape(2 * spec.inner, -1)
            b = torch.stack([bg.view(n, 8), bu.view(n, 8)], dim=1).reshape(-1) if has_bias else None
        else:
            w = torch.cat([wg, wu], dim=0)
            b = torch.cat([bg, bu]) if has_bias else None
        self.gate_up = Linear(w, b, ctx.dtype)
        self.down = Linear(tensors[prefix + "down_proj.weight"], tensors.get(prefix + "down_proj.bias"), ctx.dtype)

    takes_then = True       # the last projection may fold its output into the residual (NormAfter)
    takes_raw = True        # the first projection takes a norm's output in two pieces (RawNormed)

    def forward(self, x: torch.Tensor, batch, then=None) -> torch.Tensor:
        if self.interleave and self.gate_up.fuses_gate():
            return self.down(self.gate_up.gated(x), then=then)
        return self.down(K.silu_mul(self.gate_up(x), interleave=self.interleave), then=then)

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()


register_feed_forward("swiglu", SwiGLU)
