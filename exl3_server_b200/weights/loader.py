"""Binding checkpoint tensors to a model by name.

The model's parts say which tensors they need (``TensorSpec``: full name,
shape, class).  ``load_tensors`` compares that list with the checkpoint and
either returns every tensor or raises ONE ``WeightsError`` that lists all
missing names, all unexpected names and all wrong shapes.  The reference stops
at the first missing name (``"missing tensor <key>"``, src/model.cpp:362-366)
and lets layer norms be silently absent (src/model.cpp:408-411); here every
listed tensor is required unless its spec says ``optional`` (biases: the
reference uses a bias iff the tensor exists, src/model.cpp:370-376).

Storage rule: 16-bit floats are kept as bfloat16 (float16 is rounded to
nearest even; the reference converts the other way, src/fp16.h:70-75), a
tensor stored in 32-bit floats stays 32-bit, integer tables become int32.  The
32-bit model path widens everything to float32, which is exact.
"""
from __future__ import annotations

from dataclasses import dataclass
from fnmatch import fnmatchcase
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import TensorStore, WeightsError


@dataclass(frozen=True)
class TensorSpec:
    name: str                      # full name in the checkpoint
    shape: Tuple[int, ...]
    kind: str = "float"            # "float" or "int"
    optional: bool = False
    init: str = "normal"           # for random weights: "normal", "ones", "zeros"


_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def stored_dtype(on_disk: torch.dtype, kind: str, float_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in, given how it is stored on disk."""
    if kind == "int":
        if on_disk not in _INTS:
            raise WeightsError(f"expected an integer table, found {on_disk}")
        return torch.int32
    if on_disk not in _FLOATS:
        raise WeightsError(f"expected a float tensor, found {on_disk}")
    if float_dtype == torch.float32:
        return torch.float32
    if on_disk in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_manifest(manifest: Sequence[TensorSpec], found: Dict[str, Tuple[int, ...]],
                   ignorable: Sequence[str] = ()) -> None:
    """Raises one error naming every mismatch between ``manifest`` and the
    shapes ``found`` in a checkpoint.  Names that match one of the ``ignorable`` patterns may be there without
    being asked for (tables that some exporters store and the model recomputes, such as
    ``*.rotary_emb.inv_freq``; the reference reads by name and never looks at the rest, src/model.cpp:378-416)."""
    wanted = {s.name: s for s in manifest}
    if len(wanted) != len(manifest):
        seen, dup = set(), []
        for s in manifest:
            if s.name in seen:
                dup.append(s.name)
            seen.add(s.name)
        raise WeightsError("model lists a tensor twice: " + ", ".join(sorted(set(dup))))
    missing = [n for n, s in wanted.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in wanted and not any(fnmatchcase(n, p) for p in ignorable)]
    wrong = [(n, found[n], wanted[n].shape) for n in wanted
             if n in found and tuple(found[n]) != tuple(wanted[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = ["checkpoint does not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
            f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in sorted(wrong)))
    raise WeightsError("\n".join(lines))


def load_tensors(model_dir: str, manifest: Sequence[TensorSpec], float_dtype: torch.dtype,
                 device: torch.device | str = "cpu", ignorable: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Reads every tensor of ``manifest`` from the folder's safetensors."""
    store = TensorStore(model_dir)
    try:
        check_manifest(manifest, {n: store.shape(n) for n in store.names()}, ignorable)
        out: Dict[str, torch.Tensor] = {}
        for spec in manifest:
            if spec.name not in store.where:
                continue                      # optional and absent
            t = store.tensor(spec.name)
            try:
                dt = stored_dtype(t.dtype, spec.kind, float_dtype)
            except WeightsError as e:
                raise WeightsError(f"tensor {spec.name}: {e}")
            # copy out of the read-only mapping, convert, then place
            out[spec.name] = t.to(dtype=dt, copy=True).to(device)
        return out
    finally:
        store.close()
