"""The engine: a loaded model, its cache, and the one step function.

``Engine.step`` is the only way tokens reach the model.  Generation, trace
replay, the benchmark and the tests all drive it.  It is the reference's
``forward_multi(tokens, cache)`` (src/model.cpp:514-628) for a batch of
sequences with unequal lengths: each entry appends its tokens to its slot at
the slot's current length; prompts go in one step, then one token per step.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.kv import SequenceCache
from ..cache.pages import CacheError
from ..config.fields import ConfigError, read_config_json
from ..config.registry import resolve_architecture
from ..ops import kernels as K
from ..ops.lib import KernelLibraryError, library
from ..weights.loader import load_tensors
from .batch import StepBatch, Workspace, pack_step
from .model import Model, plan_manifest

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class StepError(ValueError):
    """A step that is refused before anything runs."""


@dataclass
class Stats:
    """What the engine's steps have had to do since it was made (or since ``reset``): the counts from which a
    caller makes rates and roofline fractions.  ``weight_bytes`` counts every weight a step uses once per step,
    ``cache_bytes`` the keys and values of the contexts that the step's tokens attend over (each sequence's
    context once per step), ``flops`` two per weight and token (the head only for the wanted rows) plus four per
    query head, head feature and visible key.  The reference reports seconds and token counts per request only
    (src/engine.h:58-75)."""
    steps: int = 0
    prompt_steps: int = 0
    decode_steps: int = 0
    tokens: int = 0
    weight_bytes: int = 0
    cache_bytes: int = 0
    flops: float = 0.0

    def reset(self) -> None:
        self.__init__()

    def minus(self, earlier: "Stats") -> "Stats":
        return Stats(**{k: getattr(self, k) - getattr(earlier, k) for k in self.__dataclass_fields__})

    def copy(self) -> "Stats":
        return Stats(**{k: getattr(self, k) for k in self.__dataclass_fields__})


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Union[str, Sequence[int], None] = "last"   # "last", "all", explicit places, or None


def resolve_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}") from None


def load_model(model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", device="cuda:0") -> Model:
    """Reads config.json, finds the architecture in the registry, checks the
    checkpoint against the plan's tensor list and builds the model."""
    from .. import models  # noqa: F401  (registers the architectures)
    dt = resolve_dtype(dtype)
    obj = read_config_json(model_dir)
    arch = resolve_architecture(obj)
    cfg = arch.config_class.from_dict(obj)
    plan = arch.build_plan(cfg)
    tensors = load_tensors(model_dir, plan_manifest(plan), dt, device, ignorable=plan.ignorable)
    model = Model(plan, tensors, dt, device)
    model.config = cfg
    return model


class Engine:
    """A model with a cache sized for ``max_tokens`` tokens (each live
    sequence's count rounded up to whole pages of 64)."""

    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None):
        if model.device.type != "cuda":
            raise KernelLibraryError("the engine runs on a CUDA device only; there is no CPU path")
        library()                                       # fail now, loudly, if the kernels are missing
        self.model = model
        self.device = model.device
        self.cache: SequenceCache = model.new_cache(max_tokens, max_slots)
        self.workspace = Workspace(self.device)
        self.decode_runners = {}
        self.steps_run = 0
        self.stats = Stats()
        self.last_generate_stats: Optional[Stats] = None
        itemsize = 4 if model.dtype == torch.float32 else 2
        self._body_params = (model.weight_bytes() - model.head.read_bytes()) // itemsize
        self._head_params = model.head.read_bytes() // itemsize
        self._cache_bytes_per_token = sum(g.bytes_per_token(itemsize) for g in self.cache.groups)
        self._score_flops_per_key = sum(4.0 * m.spec.heads * m.spec.head_dim
                                        for m in (model.blocks[e.layer].mixer for e in model.plan.schedule)
                                        if getattr(getattr(m, "spec", None), "heads", 0))

    def count_step(self, starts: Sequence[int], counts: Sequence[int], wanted: int) -> None:
        """Adds one step to ``stats``: rows that were ``starts`` long bring ``counts`` tokens each."""
        st = self.stats
        tokens = int(sum(counts))
        st.steps += 1
        if max(counts) > 1:
            st.prompt_steps += 1
        else:
            st.decode_steps += 1
        st.tokens += tokens
        st.weight_bytes += self.model.weight_bytes()
        st.cache_bytes += self._cache_bytes_per_token * int(sum(s + n for s, n in zip(starts, counts)))
        keys = sum(n * s + n * (n + 1) // 2 for s, n in zip(starts, counts))      # visible keys over the new tokens
        st.flops += 2.0 * self._body_params * tokens + 2.0 * self._head_params * wanted + self._score_flops_per_key * keys

    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", max_tokens: int = 4096, device="cuda:0",
                    max_slots: Optional[int] = None) -> "Engine":
        return cls(load_model(model_dir, dtype, device), max_tokens, max_slots)

    @property
    def stop_token_ids(self) -> List[int]:
        return list(self.model.plan.stop_token_ids)

    @property
    def cache_tokens(self) -> int:
        return self.cache.max_tokens

    @property
    def page_size(self) -> int:
        """Tokens per page of the cache: a sequence holds its length rounded up to whole pages."""
        return self.cache.page_size

    @property
    def max_positions(self) -> int:
        """The most positions a sequence may have (0: no limit given by the configuration)."""
        return int(self.model.plan.max_positions or 0)

    def generate(self, prompts, options=None, cancelled=None, on_token=None):
        """See ``engine.generate.generate``.  ``last_generate_stats`` holds the call's share of ``stats``."""
        from .generate import generate
        before = self.stats.copy()
        try:
            return generate(self, prompts, options, cancelled, on_token)
        finally:
            self.last_generate_stats = self.stats.minus(before)

    def decode_session(self, slots, max_new: int = 0):
        """Sequences that go on one token per step from a CUDA graph; see
        ``engine.decode.DecodeSession``."""
        from .decode import DecodeSession
        return DecodeSession(self, slots, None, max_new)

    # -- sequences -----------------------------------------------------------
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate(self, slot: int, new_len: int) -> None:
        """Forgets the sequence's positions from ``new_len`` on; the next step of the slot feeds the token at
        that position (the reference rewinds a cache this way to reuse a prompt's prefix,
        src/engine.cpp:244-262, src/model.cpp:630-650).  Refused for sequences with fixed-size state and for
        windowed groups that already gave back pages needed at that length."""
        self.cache.truncate(slot, new_len)

    def _decode_step(self, slots, starts, toks, wants) -> Optional[torch.Tensor]:
        """One token per entry: the recorded decode graph runs it (the same
        model code and kernels, launched from a CUDA graph)."""
        from .decode import runner_for
        runner = runner_for(self, len(slots), max(starts) + 1)
        runner.load(slots, starts, [t[0] for t in toks])
        logits = runner.run(max(starts) + 1)
        for s, st in zip(slots, starts):
            self.cache.commit(s, st + 1)
        self.steps_run += 1
        self.count_step(starts, [1] * len(slots), sum(len(w) for w in wants))
        rows = [i for i, w in enumerate(wants) for _ in w]
        if not rows:
            return None
        if rows == list(range(len(slots))):
            return logits[:len(slots)].clone()
        return logits[torch.tensor(rows, device=logits.device)]

    # -- the step ------------------------------------------------------------
    def check_kernels(self) -> None:
        """Raises if a kernel with bounded waits gave up on one since the last call (see
        ``ops.kernels.check_status``), or if the guard words around the cache's pools were overwritten.  Waits
        for the work launched so far."""
        K.check_status()
        self.cache.check_guards()

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the given tokens, as one batch, from the cache.  Returns the
        float32 logits ``[wanted, vocab]`` in the order of the entries and of
        their ``want`` lists (None when nothing is wanted)."""
        if not entries:
            raise StepError("a step needs at least one entry")
        vocab = self.model.vocab
        limit = self.model.plan.max_positions
        seen = set()
        slots, starts, toks, wants = [], [], [], []
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            try:
                start = self.cache.length(e.slot)
            except CacheError as err:
                raise StepError(str(err)) from None
            t = np.asarray(e.tokens)
            if t.ndim != 1 or t.dtype.kind not in "iu":
                t = np.asarray([int(x) for x in e.tokens], dtype=np.int64)
            if t.size == 0:
                raise StepError(f"slot {e.slot}: a step entry needs at least one token")
            bad = t[(t < 0) | (t >= vocab)]
            if bad.size:
                raise StepError(f"slot {e.slot}: token id {int(bad[0])} is outside the vocabulary of {vocab}")
            if limit and start + len(t) > limit:
                raise StepError(f"slot {e.slot}: {start + len(t)} positions exceed max_position_embeddings {limit}")
            if e.want is None:
                w: List[int] = []
            elif isinstance(e.want, str):
                if e.want == "last":
                    w = [len(t) - 1]
                elif e.want == "all":
                    w = list(range(len(t)))
                else:
                    raise StepError(f"want must be 'last', 'all', a list of places or None, got {e.want!r}")
            else:
                w = [int(x) for x in e.want]
                if any(not 0 <= x < len(t) for x in w):
                    raise StepError(f"slot {e.slot}: wanted place outside the {len(t)} tokens of this step")
                if len(set(w)) != len(w):
                    raise StepError(f"slot {e.slot}: a place is wanted twice in one step")
            slots.append(e.slot)
            starts.append(start)
            toks.append(t)
            wants.append(w)
        self.cache.reserve({s: st + len(t) for s, st, t in zip(slots, starts, toks)})
        if all(len(t) == 1 for t in toks):
            return self._decode_step(slots, starts, toks, wants)
        batch = pack_step(slots, starts, toks, wants, self.cache.block_tables(slots), self.workspace, self.device)
        logits = self.model.forward(batch, self.cache)
        for s, st, t in zip(slots, starts, toks):
            self.cache.commit(s, st + len(t))
        self.steps_run += 1
        self.count_step(starts, [len(t) for t in toks], sum(len(w) for w in wants))
        return logits
