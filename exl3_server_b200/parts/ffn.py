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
        w = torch.cat([tensors[prefix + "gate_proj.weight"].to(ctx.dtype),
                       tensors[prefix + "up_proj.weight"].to(ctx.dtype)], dim=0)
        bg, bu = tensors.get(prefix + "gate_proj.bias"), tensors.get(prefix + "up_proj.bias")
        b = None
        if bg is not None or bu is not None:
            z = torch.zeros(spec.inner, dtype=ctx.dtype, device=w.device)
            b = torch.cat([(bg.to(ctx.dtype) if bg is not None else z), (bu.to(ctx.dtype) if bu is not None else z)])
        self.gate_up = Linear(w, b, ctx.dtype)
        self.down = Linear(tensors[prefix + "down_proj.weight"], tensors.get(prefix + "down_proj.bias"), ctx.dtype)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        return self.down(K.silu_mul(self.gate_up(x)))

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()


register_feed_forward("swiglu", SwiGLU)
