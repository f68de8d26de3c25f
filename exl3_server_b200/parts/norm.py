"""RMSNorm fused with the residual add.

``r = h * rsqrt(mean(h^2) + eps) * w`` with the weight multiplying directly
(no ``1 + w``), as the reference's ``mx::fast::rms_norm`` calls use it
(src/model.cpp:556, 582, 589).  The sum of squares, the reciprocal root and the
residual add ``h += scale * y`` are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, ResidualStream
from .registry import register_norm
from .spec import NormSpec


class RMSNorm:
    @staticmethod
    def tensor_specs(spec: NormSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + "weight", (spec.width,), init="ones")]

    def __init__(self, spec: NormSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        w = tensors[prefix + "weight"]
        # a weight stored in 32-bit stays 32-bit; the kernel reads either
        self.weight = w.contiguous() if w.dtype == torch.float32 else w.to(ctx.dtype).contiguous()
        self.out_dtype = ctx.dtype

    offers_raw = True

    def add_norm(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                 out_scale: float = 1.0, raw_ok: bool = False):
        """``raw_ok``: the caller's next projection takes a ``RawNormed`` (the output in two pieces, left by the
        projection before this norm) as well as a tensor."""
        left = stream.take_normed(self)
        if left is not None:
            if rows is None and raw_ok and out_scale == 1.0:
                return left
            return left.materialize(out_scale, rows)
        y, s = stream.take()
        return K.add_rmsnorm(stream.h, y, s, self.weight, self.spec.eps, self.out_dtype,
                             out_scale=out_scale, rows=rows)

    def fuse_args(self):
        """``(weight, eps, width)`` for a projection kernel that prepares this norm (see ``NormAfter``)."""
        return self.weight, self.spec.eps, self.spec.width

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()


register_norm("rms", RMSNorm)
