"""Choosing how a batch of logit rows is sampled.

Rows that are all greedy, or all plain temperature without filters or
penalties, are sampled on the device by the argmax / inverse-CDF kernels and
only the chosen ids cross to the host.  Anything else (top-k, top-p, min-p,
penalties, or a mixed batch) is sampled on the host by the reference's
algorithm, which is where the reference always samples (src/model.cpp:667-757).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .host import sample_token
from .options import SampleOptions, SplitMix64


class RowSampler:
    """Sampling state of one request: its options, generator and context."""

    def __init__(self, opt: SampleOptions, request_index: int, prompt: Sequence[int]):
        self.opt = opt
        self.rng = SplitMix64(opt.seed + request_index)
        self.context: List[int] = list(prompt)


def sample_rows(logits: torch.Tensor, rows: Sequence[RowSampler],
                device_argmax: Optional[torch.Tensor] = None) -> List[int]:
    """One token per row of ``logits`` ``[len(rows), vocab]`` (float32).
    ``device_argmax`` is the argmax of each row when the step already
    computed it on the device."""
    if logits.shape[0] != len(rows):
        raise ValueError(f"{logits.shape[0]} logit rows for {len(rows)} requests")
    if logits.is_cuda and not any(r.opt.has_penalties for r in rows):
        from ..ops import kernels as K
        if all(r.opt.greedy for r in rows):
            ids = device_argmax if device_argmax is not None else K.argmax(logits)
            picked = ids.cpu().tolist()
            from ..engine.decode import TRANSFERRED
            TRANSFERRED["d2h"] += ids.numel() * 4
            for r, t in zip(rows, picked):
                r.context.append(t)
            return picked
        temps = {r.opt.temperature for r in rows}
        if len(temps) == 1 and not any(r.opt.greedy or r.opt.has_filters for r in rows):
            u = torch.tensor([r.rng.uniform01() for r in rows], dtype=torch.float32).to(logits.device)
            picked = K.sample_temperature(logits, u, temps.pop()).cpu().tolist()
            for r, t in zip(rows, picked):
                r.context.append(t)
            return picked
    host = logits.detach().to(torch.float32).cpu().numpy()
    out = []
    for i, r in enumerate(rows):
        t = sample_token(host[i], r.opt, r.context, r.rng)
        r.context.append(t)
        out.append(t)
    return out
