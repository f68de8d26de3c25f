"""Token embedding and output head.

Embedding: ``h0[t] = E[id_t] * scale`` (the gather is src/model.cpp:529; the
scale is MiniCPM's ``scale_emb``).  Head: ``logits = (norm(h) / divisor) W^T``
in float32, computed only for the rows that were asked for (the reference
computes every row, src/model.cpp:589-592); ``W`` is the embedding table when
the head is tied.

Both are registered part kinds like the others (``"table"`` and ``"linear"``).  An embedding of another kind has
``tensor_specs(spec)``, ``__init__(spec, tensors, ctx)`` and ``forward(token_ids) -> ResidualStream``; a head has
``tensor_specs(spec)``, ``__init__(spec, tensors, embedding, ctx)``, ``forward(stream, final_norm, rows) ->
float32 logits [rows, vocab]`` and ``read_bytes()``, the weight bytes a step reads.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, ResidualStream
from .linear import Linear
from .registry import register_embedding, register_head
from .spec import EmbeddingSpec, HeadSpec


class Embedding:
    @staticmethod
    def tensor_specs(spec: EmbeddingSpec) -> List[TensorSpec]:
        return [TensorSpec(spec.name, (spec.vocab, spec.width))]

    def __init__(self, spec: EmbeddingSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec = spec
        self.table = tensors[spec.name].to(ctx.dtype).contiguous()

    def forward(self, token_ids: torch.Tensor) -> ResidualStream:
        return ResidualStream(K.embed(token_ids, self.table, float(self.spec.scale)))

    def weight_bytes(self) -> int:
        return self.table.numel() * self.table.element_size()


class Head:
    @staticmethod
    def tensor_specs(spec: HeadSpec) -> List[TensorSpec]:
        if spec.tied:
            return []
        # tied None: the configuration does not say; a head of its own is used when the checkpoint has one
        return [TensorSpec(spec.name, (spec.vocab, spec.width), optional=spec.tied is None)]

    def __init__(self, spec: HeadSpec, tensors: Dict[str, torch.Tensor], embedding: Embedding, ctx: BuildContext):
        self.spec = spec
        self.tied = spec.tied if spec.tied is not None else spec.name not in tensors
        weight = embedding.table if self.tied else tensors[spec.name]
        self.linear = Linear(weight, None, ctx.dtype)
        if self.tied:
            self.linear.weight = embedding.table          # one copy in memory

    def forward(self, stream: ResidualStream, final_norm, rows: Optional[torch.Tensor]) -> torch.Tensor:
        r = final_norm.add_norm(stream, rows=rows, out_scale=1.0 / float(self.spec.input_divisor))
        return self.linear(r, out_dtype=torch.float32)

    def weight_bytes(self) -> int:
        """Bytes this part holds beyond the embedding's."""
        return 0 if self.tied else self.linear.weight_bytes()

    def read_bytes(self) -> int:
        """Weight bytes a step reads for the logits (a tied head reads the embedding table)."""
        return self.linear.weight_bytes()


register_embedding("table", Embedding)
register_head("linear", Head)
