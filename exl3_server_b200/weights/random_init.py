"""Random-weights mode: a model folder from a configuration and a seed.

``write_random_model`` writes ``config.json`` and ``model.safetensors`` for any
registered architecture.  Each tensor has its own generator seeded from the
seed and the tensor's name, so a tensor's values do not depend on which other
tensors exist.  Matrices are N(0, std); norm weights are ``1 + N(0, norm_std)``
or, with ``norm_std=None``, N(0, std) like everything else; optional tensors
(biases) are written only when ``with_optional`` is set.  The reference has no
such mode; its tests seed ``mt19937`` by hand (tests/mla_incremental_test.cpp:21-41).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Iterator, Optional, Sequence, Tuple

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = int.from_bytes(hashlib.sha256(name.encode("utf-8")).digest()[:8], "little")
    return (seed * 0x9E3779B97F4A7C15 + h) & 0x7FFFFFFFFFFFFFFF


def random_tensors(manifest: Sequence[TensorSpec], seed: int, std: float = 0.02,
                   norm_std: Optional[float] = 0.01, dtype: torch.dtype = torch.bfloat16,
                   with_optional: bool = False, device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    for spec in manifest:
        if spec.optional and not with_optional:
            continue
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, spec.name))
        if spec.kind == "int":
            yield spec.name, torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        x = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
        if spec.init == "ones":
            x = 1.0 + x * norm_std if norm_std is not None else x * std
        else:                                           # "normal", and biases when asked for
            x = x * std
        yield spec.name, x.to(dtype)


def write_random_model(config: Any, folder: str, seed: int, std: float = 0.02,
                       norm_std: Optional[float] = 0.01, dtype: torch.dtype = torch.bfloat16,
                       with_optional: bool = False) -> str:
    """Writes ``folder/config.json`` and ``folder/model.safetensors`` for the
    typed configuration ``config`` (its class must be registered)."""
    from .. import models  # noqa: F401
    from ..config.registry import resolve_architecture
    from ..engine.model import plan_manifest
    obj: Dict[str, Any] = config.to_dict()
    arch = resolve_architecture(obj)
    plan = arch.build_plan(config)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(obj, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(plan_manifest(plan), seed, std, norm_std, dtype, with_optional),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
