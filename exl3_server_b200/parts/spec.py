"""Descriptions of parts: plain data that a configuration is turned into.

An architecture's plan builder (``models/<arch>.py``) reads its typed
configuration and writes one ``ModelPlan``.  The plan holds a ``LayerSpec`` per
layer; each names a mixer, a feed-forward, two norms and a block arrangement
with all their sizes and constants, so that layers of one model may differ.
Nothing below this level looks at a configuration again.  The precedent is the
reference's per-layer ``LayerPlan`` (src/model.h:40-45).

``ModelPlan.schedule`` is the order in which layers run.  It is data: an entry
names the layer whose weights run, and optionally the earlier entry whose cache
it reads instead of owning one, so a layer may run twice and a layer may read
another layer's keys and values.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class NormSpec:
    kind: str                     # registered norm name, e.g. "rms"
    width: int
    eps: float
    params: Dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class PositionSpec:
    kind: str                     # registered position encoding, e.g. "rope", "none"
    dims: int                     # rotated features per head
    theta: float = 10000.0
    scale: float = 1.0            # positions are multiplied by this (1 = plain)
    params: Dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class MixerSpec:
    kind: str                     # registered mixer name, e.g. "attention"
    width: int                    # model width going in and out
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0               # 0: every earlier key; n: the last n keys
    softmax_scale: Optional[float] = None   # None: head_dim ** -0.5
    position: Optional[PositionSpec] = None
    params: Dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                     # registered feed-forward name, e.g. "swiglu"
    width: int
    inner: int
    params: Dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which parts, in which arrangement, under which tensor names."""
    arrangement: str              # registered block arrangement, e.g. "prenorm"
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    residual_scale: float         # sublayer outputs are multiplied by this before the add
    # tensor-name prefixes in the checkpoint, by role
    names: Dict[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                            # index into ModelPlan.layers
    cache_from: Optional[int] = None      # schedule index whose cache this entry reads


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab: int
    width: int
    scale: float
    name: str
    kind: str = "table"           # registered embedding name
    params: Dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class HeadSpec:
    vocab: int
    width: int
    input_divisor: float          # the normed hidden state is divided by this
    tied: Optional[bool]          # True: the embedding table is the head's weight; None: it is when the
                                  # checkpoint has no tensor called ``name``
    name: str
    kind: str = "linear"          # registered head name
    params: Dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass
class ModelPlan:
    architecture: str
    embedding: EmbeddingSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: NormSpec
    final_norm_name: str
    head: HeadSpec
    max_positions: int            # 0: not limited by the configuration
    stop_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    # patterns (``fnmatch``) of tensor names that a checkpoint of this architecture may carry and the model
    # does not read; any other tensor the parts did not ask for is an error
    ignorable: List[str] = field(default_factory=list)

    def validate(self) -> None:
        n = len(self.layers)
        if not self.schedule:
            raise ValueError("plan: empty schedule")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"plan: schedule[{i}] names layer {e.layer}, model has {n}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ValueError(
                        f"plan: schedule[{i}] reads the cache of entry {e.cache_from}, "
                        "which must be an earlier entry")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(
                        f"plan: schedule[{i}] reads entry {e.cache_from}, which owns no cache")
