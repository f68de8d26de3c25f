"""Tiny configurations, traces and comparison helpers shared by the tests."""
from __future__ import annotations

import random
from typing import Dict, List, Sequence

import numpy as np
import torch

from exl3_server_b200 import LlamaConfig, write_random_model

# Tiny configurations that differ in every size and option.
#  A: MiniCPM-style; grouped heads 4/2, head 16, tied head, all three scale constants.
#  B: plain Llama; one kv head, head 32, untied, other theta and eps, no scaling.
#  D: heads of 64 (the tensor-core attention's shape), width 136, vocabulary 301.
#  E: grouped heads of 128 (see below).
#  C: odd sizes: width 96, 6/3 heads of 48, vocabulary 263, a window of 24 keys on
#     layers 0 and 2 (full attention on 1 and 3), biases on every projection.
TINY: Dict[str, dict] = {
    "A": dict(cfg=LlamaConfig(
        hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        intermediate_size=176, vocab_size=256, tie_word_embeddings=True, rope_theta=10000.0,
        rms_norm_eps=1e-5, scale_emb=12.0, scale_depth=1.4, dim_model_base=32, max_position_embeddings=512,
        eos_token_id=[2], model_type="minicpm", architectures=["MiniCPMForCausalLM"]),
        norm_std=0.01, biases=False),
    "B": dict(cfg=LlamaConfig(
        hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=1, head_dim=32,
        intermediate_size=352, vocab_size=384, tie_word_embeddings=False, rope_theta=500000.0,
        rms_norm_eps=1e-6, max_position_embeddings=1024, eos_token_id=[0, 383]),
        norm_std=0.2, biases=False),
    "C": dict(cfg=LlamaConfig(
        hidden_size=96, num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
        intermediate_size=200, vocab_size=263, tie_word_embeddings=False, rope_theta=2500.0,
        rms_norm_eps=3e-6, scale_emb=3.0, scale_depth=2.0, dim_model_base=48, max_position_embeddings=2048,
        sliding_window=24,
        layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"]),
        norm_std=0.05, biases=True),
    # D: heads of 64, the shape the tensor-core kernels take; a window on the last layer.
    "D": dict(cfg=LlamaConfig(
        hidden_size=136, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
        intermediate_size=208, vocab_size=301, tie_word_embeddings=True, rope_theta=100000.0,
        rms_norm_eps=1e-5, scale_emb=2.0, scale_depth=1.0, dim_model_base=68, max_position_embeddings=4096,
        sliding_window=80, layer_types=["full_attention", "sliding_attention"]),
        norm_std=0.1, biases=False),
    # E: grouped heads of 128 (6 query heads on 2), the tensor-core kernels' other shape; untied head, a window
    # of 150 keys on the first layer.
    "E": dict(cfg=LlamaConfig(
        hidden_size=200, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
        intermediate_size=272, vocab_size=331, tie_word_embeddings=False, rope_theta=500000.0,
        rms_norm_eps=2e-5, max_position_embeddings=4096,
        sliding_window=150, layer_types=["sliding_attention", "full_attention"]),
        norm_std=0.15, biases=False),
}


def make_folder(name: str, folder: str, std: float = 0.08) -> str:
    t = TINY[name]
    # std 0.08 instead of the usual 0.02 makes attention scores of order one, so that a wrong
    # mask, position or cache slot changes the logits by far more than rounding does; norm
    # weights are 1 + N(0, norm_std) (0.2 is the reference's own choice in its synthetic
    # tests, tests/mla_incremental_test.cpp:42-77)
    return write_random_model(t["cfg"], folder, seed=1234 + ord(name), std=std, norm_std=t["norm_std"],
                              dtype=torch.bfloat16, with_optional=t["biases"])


def random_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


# -- traces (the JSON step objects that bin/trace_run reads) -----------------

def whole_trace(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone, all its tokens in one step, every logit wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail_trace(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Each request alone: all but the last ``tail`` tokens in one step, then one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(0, len(toks) - tail)
        if head:
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                          "end": []})
            n += 1
        for i in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            n += 1
    return steps


def batched_trace(requests: Dict[str, List[int]], batches: Sequence[Sequence[str]],
                  prompt_len: Dict[str, int]) -> List[dict]:
    """Batches one after another.  A batch's requests start together with
    their first ``prompt_len`` tokens in one step, then go on one token per
    step (the trace's own tokens); a request whose tokens run out ends."""
    steps, n = [], 0
    for batch in batches:
        fed = {rid: prompt_len[rid] for rid in batch}
        entries = [{"id": rid, "tokens": requests[rid][:fed[rid]], "want": list(range(fed[rid]))} for rid in batch]
        live = list(batch)
        while True:
            ending = [rid for rid in live if fed[rid] >= len(requests[rid])]
            steps.append({"step": n, "entries": entries, "end": ending})
            n += 1
            live = [rid for rid in live if rid not in ending]
            if not live:
                break
            entries = [{"id": rid, "tokens": [requests[rid][fed[rid]]], "want": [0]} for rid in live]
            for rid in live:
                fed[rid] += 1
    return steps


def run_trace(engine, steps: List[dict]) -> Dict[str, np.ndarray]:
    """Runs trace steps in-process through the replay tool's runner and
    gathers, per request, the logits of every position ``[n, vocab]``."""
    from exl3_server_b200.replay import TraceRunner
    runner = TraceRunner(engine)
    got: Dict[str, Dict[int, np.ndarray]] = {}
    fed: Dict[str, int] = {}
    for msg in steps:
        logits = runner.run_step(msg)
        arr = None if logits is None else logits.float().cpu().numpy()
        row = 0
        for e in msg["entries"]:
            base = fed.get(e["id"], 0)
            for w in e.get("want", []):
                got.setdefault(e["id"], {})[base + w] = arr[row]
                row += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in msg.get("end", []):
            fed.pop(rid, None)                      # the same id may come again in a later batch
    engine.cache.check()
    return {rid: np.stack([rows[i] for i in sorted(rows)]) for rid, rows in got.items()}


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """Largest absolute difference relative to the largest reference value."""
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) / max(1e-30, np.max(np.abs(b))))


# Bounds on rounding, fixed before the first GPU run and never widened:
#  float32: every reduction is float32 (unit roundoff 6e-8) over at most a few
#  thousand terms, through at most 4 layers: 1e-5 of the largest logit leaves
#  two orders of margin and is far below any indexing or masking fault (>= 1e-2).
#  bfloat16: activations are rounded to 8 bits (unit roundoff 3.9e-3) after every
#  kernel; about ten roundings per layer feed a logit, so a few 1e-2 of the
#  largest logit; 5e-2 bounds it, faults show as 0.3 and more.
TOL = {"float32": 1e-5, "bfloat16": 5e-2}
