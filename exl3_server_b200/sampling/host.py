"""The reference's sampler on the host, step for step (``sample_token``,
src/model.cpp:667-757): penalties over the context, then greedy, or the
``max(top_k, 2048)`` most probable candidates in descending order, temperature
softmax (float32 terms, float64 sums), min-p, top-k, top-p, and an
inverse-CDF draw with one uniform number from the request's generator."""
from __future__ import annotations

from collections import Counter
from typing import Sequence

import numpy as np

from .options import SampleOptions, SplitMix64


def apply_penalties(logits: np.ndarray, opt: SampleOptions, context: Sequence[int]) -> None:
    """In place (src/model.cpp:672-686)."""
    if not opt.has_penalties:
        return
    n = logits.shape[0]
    counts = Counter(t for t in context if 0 <= t < n)
    for t, c in counts.items():
        x = np.float32(logits[t])
        if opt.repetition_penalty != 1.0:
            r = np.float32(opt.repetition_penalty)
            x = x / r if x > 0 else x * r
        if opt.presence_penalty != 0.0:
            x = x - np.float32(opt.presence_penalty)
        if opt.frequency_penalty != 0.0:
            x = x - np.float32(opt.frequency_penalty) * np.float32(c)
        logits[t] = x


def sample_token(logits: np.ndarray, opt: SampleOptions, context: Sequence[int], rng: SplitMix64) -> int:
    logits = np.array(logits, dtype=np.float32, copy=True)
    n = logits.shape[0]
    apply_penalties(logits, opt, context)
    if opt.temperature <= 0.0:
        return int(np.argmax(logits))                     # first maximum (src/model.cpp:688-696)
    cap = max(opt.top_k if opt.top_k > 0 else 0, 2048)   # src/model.cpp:698
    m = min(n, cap)
    if m < n:
        # equal logits rank by index, the smaller first (the reference's partial sort leaves their order open;
        # the device sampler ranks them the same way)
        neg = -logits
        kth = np.partition(neg, m - 1)[m - 1]
        above = np.nonzero(neg < kth)[0]
        ties = np.nonzero(neg == kth)[0][:m - above.size]
        part = np.sort(np.concatenate([above, ties]))
        idx = part[np.argsort(neg[part], kind="stable")]
    else:
        idx = np.argsort(-logits, kind="stable")
    inv_t = np.float32(1.0) / np.float32(opt.temperature)
    maxl = logits[idx[0]] * inv_t
    probs = np.exp(logits[idx] * inv_t - maxl).astype(np.float32)
    total = float(np.sum(probs, dtype=np.float64))
    if not total > 0.0:
        return int(idx[0])
    keep = m
    if opt.min_p > 0.0:                                   # src/model.cpp:724-733
        thresh = float(opt.min_p) * (float(probs[0]) / total)
        below = np.nonzero(probs.astype(np.float64) / total < thresh)[0]
        keep = int(below[0]) if below.size else m
        keep = max(keep, 1)
    if 0 < opt.top_k < keep:                              # src/model.cpp:735
        keep = opt.top_k
    if opt.top_p < 1.0:                                   # src/model.cpp:737-746
        acc = np.cumsum(probs[:keep], dtype=np.float64) / total
        hit = np.nonzero(acc >= float(opt.top_p))[0]
        keep = max(1, int(hit[0]) + 1 if hit.size else keep)
    kept = probs[:keep].astype(np.float64)
    r = rng.uniform01() * float(np.sum(kept))             # src/model.cpp:748-756
    chosen = keep - 1
    for i in range(keep):
        r -= kept[i]
        if r <= 0.0:
            chosen = i
            break
    return int(idx[chosen])
