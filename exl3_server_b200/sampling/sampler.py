"""Choosing how a batch of logit rows is sampled.

Rows that are all greedy take the argmax kernel.  Everything else that the
device sampler covers (temperature with top-k up to its cap, top-p, min-p and
the penalties over the context) is sampled on the device by the reference's
algorithm (``csrc/sampling_filtered.cu``): only the options, the uniform numbers
and the chosen ids cross between host and device.  ``host.sample_token`` is the
same algorithm on the host (src/model.cpp:667-757), for logits that are not on
the device and for ``top_k`` above the cap; the tests hold the two against
each other.
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
        self._counts: Optional[torch.Tensor] = None      # int32 [vocab] on the device: how often each token occurs
        self._counted = 0                                # tokens of the context that the counts hold

    def device_counts(self, vocab: int, device) -> torch.Tensor:
        """The context's token counts on the device, for the penalties: made from the whole context when first
        asked for, then kept up by the sampler's own kernel (``counted``) or from the context's new tokens."""
        if self._counts is None:
            self._counts = torch.zeros(vocab, dtype=torch.int32, device=device)
        if self._counted < len(self.context):
            new = torch.tensor([t for t in self.context[self._counted:] if 0 <= t < vocab], dtype=torch.int64)
            if new.numel():
                self._counts.index_add_(0, new.to(device), torch.ones(new.numel(), dtype=torch.int32, device=device))
            self._counted = len(self.context)
        return self._counts

    def counted(self, n: int = 1) -> None:
        """The device has added the next ``n`` tokens of the context to the counts itself."""
        self._counted += n


def on_device(logits: torch.Tensor, rows: Sequence[RowSampler]) -> bool:
    """Whether ``launch_on_device`` takes this batch."""
    if not logits.is_cuda:
        return False
    from ..ops import kernels as K
    return all(r.opt.top_k <= K.sample_filtered_cap() for r in rows)


def launch_on_device(logits: torch.Tensor, rows: Sequence[RowSampler]) -> torch.Tensor:
    """Starts the sampling of one token per row on the device and returns the ids (int32 on the device)
    without waiting for them.  The generators advance now; the tokens join the rows' contexts when the caller
    has read them (``record``).  The penalties' token counts are kept up on the device."""
    from ..engine.decode import TRANSFERRED
    from ..ops import kernels as K
    R, V = logits.shape
    counts = None
    if any(r.opt.has_penalties for r in rows):
        logits = logits.clone()                          # the step's own buffer stays as the model left it
        counts = torch.tensor([r.device_counts(V, logits.device).data_ptr() if r.opt.has_penalties else 0
                               for r in rows], dtype=torch.int64).to(logits.device)
        params = torch.tensor([[r.opt.repetition_penalty, r.opt.presence_penalty, r.opt.frequency_penalty]
                               for r in rows], dtype=torch.float32)
        TRANSFERRED["h2d"] += counts.numel() * 8 + params.numel() * 4
        K.sample_penalties(logits, counts, params.to(logits.device))
    # a greedy row draws no number from its generator, as on the host
    opts = torch.tensor([[r.opt.temperature, r.opt.top_k, r.opt.top_p, r.opt.min_p,
                          0.0 if r.opt.greedy else r.rng.uniform01()] for r in rows], dtype=torch.float64)
    ids = K.sample_filtered(logits, opts.to(logits.device))
    if counts is not None:
        K.sample_count(counts, ids, V)                   # the chosen tokens join the counts without a trip to the host
        for r in rows:
            if r.opt.has_penalties:
                r.counted()
    TRANSFERRED["h2d"] += opts.numel() * 8
    return ids


def record(rows: Sequence[RowSampler], picked: Sequence[int]) -> None:
    """The rows' sampled tokens, read by the host, join their contexts."""
    for r, t in zip(rows, picked):
        r.context.append(int(t))


def sample_rows(logits: torch.Tensor, rows: Sequence[RowSampler],
                device_argmax: Optional[torch.Tensor] = None) -> List[int]:
    """One token per row of ``logits`` ``[len(rows), vocab]`` (float32).
    ``device_argmax`` is the argmax of each row when the step already
    computed it on the device."""
    if logits.shape[0] != len(rows):
        raise ValueError(f"{logits.shape[0]} logit rows for {len(rows)} requests")
    picked: Optional[List[int]] = None
    if logits.is_cuda:
        from ..ops import kernels as K
        if all(r.opt.greedy and not r.opt.has_penalties for r in rows):
            ids = device_argmax if device_argmax is not None else K.argmax(logits)
            picked = ids.cpu().tolist()
            from ..engine.decode import TRANSFERRED
            TRANSFERRED["d2h"] += ids.numel() * 4
        elif on_device(logits, rows):
            ids = launch_on_device(logits.to(torch.float32), rows)
            picked = ids.cpu().tolist()
            from ..engine.decode import TRANSFERRED
            TRANSFERRED["d2h"] += ids.numel() * 4
    if picked is None:
        host = logits.detach().to(torch.float32).cpu().numpy()
        picked = [sample_token(host[i], r.opt, r.context, r.rng) for i, r in enumerate(rows)]
    record(rows, picked)
    return picked
