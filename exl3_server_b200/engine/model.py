"""A model assembled from a plan: embedding, layers built from registered
parts, the schedule that orders them, the final norm and the head.

The forward pass runs exactly the tokens of a ``StepBatch`` against the cache
and returns float32 logits for the wanted rows.  It is the reference's
``Model::forward_multi`` (src/model.cpp:514-628) for a packed batch of
sequences with a paged cache.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.kv import SequenceCache
from ..parts.base import BuildContext, KVRequest, StateRequest
from ..parts.registry import (arrangement_class, embedding_class, feed_forward_class, head_class, mixer_class,
                              norm_class)
from ..parts.spec import ModelPlan
from ..weights.loader import TensorSpec
from .batch import StepBatch


def plan_manifest(plan: ModelPlan) -> List[TensorSpec]:
    """Every tensor the plan's parts will ask for, by checkpoint name."""
    specs: List[TensorSpec] = list(embedding_class(plan.embedding.kind).tensor_specs(plan.embedding))
    for layer in plan.layers:
        specs += mixer_class(layer.mixer.kind).tensor_specs(layer.mixer, layer.names["mixer"])
        specs += feed_forward_class(layer.feed_forward.kind).tensor_specs(layer.feed_forward,
                                                                         layer.names["feed_forward"])
        specs += norm_class(layer.mixer_norm.kind).tensor_specs(layer.mixer_norm, layer.names["mixer_norm"])
        specs += norm_class(layer.feed_forward_norm.kind).tensor_specs(layer.feed_forward_norm,
                                                                      layer.names["feed_forward_norm"])
    specs += norm_class(plan.final_norm.kind).tensor_specs(plan.final_norm, plan.final_norm_name)
    specs += head_class(plan.head.kind).tensor_specs(plan.head)
    return specs


class Model:
    def __init__(self, plan: ModelPlan, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device):
        plan.validate()
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        ctx = BuildContext(dtype=dtype, device=self.device)
        self.embedding = embedding_class(plan.embedding.kind)(plan.embedding, tensors, ctx)
        self.blocks = []
        for layer in plan.layers:
            mixer = mixer_class(layer.mixer.kind)(layer.mixer, tensors, layer.names["mixer"], ctx)
            ff = feed_forward_class(layer.feed_forward.kind)(layer.feed_forward, tensors,
                                                             layer.names["feed_forward"], ctx)
            n1 = norm_class(layer.mixer_norm.kind)(layer.mixer_norm, tensors, layer.names["mixer_norm"], ctx)
            n2 = norm_class(layer.feed_forward_norm.kind)(layer.feed_forward_norm, tensors,
                                                          layer.names["feed_forward_norm"], ctx)
            self.blocks.append(arrangement_class(layer.arrangement)(layer, mixer, ff, n1, n2))
        self.final_norm = norm_class(plan.final_norm.kind)(plan.final_norm, tensors, plan.final_norm_name, ctx)
        self.head = head_class(plan.head.kind)(plan.head, tensors, self.embedding, ctx)
        self.vocab = plan.head.vocab

    def cache_requests(self) -> List[Tuple[Optional[KVRequest], Optional[StateRequest], Optional[int]]]:
        out = []
        for e in self.plan.schedule:
            m = self.blocks[e.layer].mixer
            out.append((m.cache_request(), m.state_request(), e.cache_from))
        return out

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None) -> SequenceCache:
        return SequenceCache(self.cache_requests(), max_tokens, dtype=self.dtype, device=self.device,
                             max_slots=max_slots)

    def forward(self, batch: StepBatch, cache: SequenceCache) -> Optional[torch.Tensor]:
        stream = self.embedding.forward(batch.token_ids)
        sched = self.plan.schedule
        for i, e in enumerate(sched):
            block = self.blocks[e.layer]
            kv, state = cache.view(i, batch.block_tables), cache.state_of(i)
            if getattr(block, "takes_after", False):
                # the norm that the next block applies first, so that this block's last projection may apply it
                nxt = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None
                block.forward(stream, batch, kv, state, after=getattr(nxt, "mixer_norm", None))
            else:
                block.forward(stream, batch, kv, state)
        if batch.n_wanted == 0:
            return None
        return self.head.forward(stream, self.final_norm, batch.want_rows)

    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads (each matrix once; a tied head
        reads the embedding table)."""
        n = sum(self.blocks[e.layer].weight_bytes() for e in self.plan.schedule)
        n += self.final_norm.weight_bytes()
        n += self.head.read_bytes()
        return n
