"""The engine against the plain implementation, for every way of cutting the
same requests into steps: whole, with the last 32 tokens one by one, and in
batches of unequal lengths whose shorter requests end earlier, in float32 and
in bfloat16, on tiny configurations that differ in every size and option."""
import numpy as np
import pytest
import torch

from helpers import TINY, TOL, batched_trace, random_requests, rel_err, run_trace, tail_trace, whole_trace
from plain_llama import PlainModel

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 9, 13, 70, 131], "B": [1, 17, 40, 64, 97], "C": [3, 33, 64, 65, 150],
           "D": [2, 64, 129, 200, 333], "E": [1, 63, 130, 257, 300]}
_plain_cache = {}


def plain_logits(folder, requests):
    key = (folder, tuple(sorted((k, tuple(v)) for k, v in requests.items())))
    if key not in _plain_cache:
        pm = PlainModel(folder)
        _plain_cache[key] = {rid: pm.logits(t).numpy() for rid, t in requests.items()}
    return _plain_cache[key]


def engine_for(folder, dtype, max_tokens=1024):
    from exl3_server_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens)


def check(got, want, dtype, what):
    assert set(got) == set(want)
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        assert np.isfinite(got[rid]).all(), (what, rid)
        err = rel_err(got[rid], want[rid])
        if err > TOL[dtype]:
            per_pos = np.max(np.abs(got[rid] - want[rid]), axis=1) / np.max(np.abs(want[rid]))
            first = int(np.argmax(per_pos > TOL[dtype]))
            raise AssertionError(f"{what}: request {rid} (length {len(per_pos)}) differs from the plain "
                                 f"implementation by {err:.3e} (bound {TOL[dtype]:.0e}); first wrong position {first}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_whole_tail_and_batched(model_folders, name, dtype):
    folder = model_folders[name]
    vocab = TINY[name]["cfg"].vocab_size
    requests = random_requests(vocab, LENGTHS[name], seed=7)
    want = plain_logits(folder, requests)
    eng = engine_for(folder, dtype)

    check(run_trace(eng, whole_trace(requests)), want, dtype, "whole")
    check(run_trace(eng, tail_trace(requests, 32)), want, dtype, "last 32 one by one")

    ids = list(requests)
    # two batches after one another, so that slots and pages are used again; prompts of
    # unequal lengths (one of a single token), the rest of each request fed one token a step
    batches = [[ids[4], ids[0], ids[2]], [ids[1], ids[3], ids[0]]]
    prompt_len = {rid: max(1, len(requests[rid]) - k) for rid, k in zip(ids, (3, 16, 0, 40, 33))}
    check(run_trace(eng, batched_trace(requests, batches, prompt_len)),
          {rid: want[rid] for b in batches for rid in b}, dtype, "batched")
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("name", list(TINY))
def test_float32_cuttings_agree_closely(model_folders, name):
    """In float32 every reduction has an order that depends only on the
    token's own position, so the three cuttings agree to the last bits."""
    folder = model_folders[name]
    requests = random_requests(TINY[name]["cfg"].vocab_size, LENGTHS[name], seed=11)
    eng = engine_for(folder, "float32")
    a = run_trace(eng, whole_trace(requests))
    b = run_trace(eng, tail_trace(requests, 32))
    for rid in requests:
        assert rel_err(b[rid], a[rid]) <= 1e-6, rid
