"""Schedules that only large runs reach, checked against the plain implementation: decode batches of 8 to 64
rows whose requests end at different steps (through the step function and through a decode session), a second
batch on the same engine, contexts beyond 4,096 tokens, rewinding a sequence and feeding other tokens, two
users of decode runners of one shape, and a recorded step that runs again after a later one needed more
scratch memory.  The reference's counterparts: joins and leaves of its batched loop
(tests/glm5_batch_test.cpp:172-293) and prefix reuse by rewinding (src/engine.cpp:244-262)."""
import dataclasses
import random

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, batched_trace, random_requests, rel_err, run_trace
from plain_llama import PlainModel

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype, max_tokens=2048, max_slots=None):
    from exl3_server_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, max_slots=max_slots)


def unequal_requests(vocab, n, seed, longest_tail):
    """n requests: prompts of 1 to 90 tokens (1, 64 and 65 among them), then 2 to ``longest_tail`` tokens one by
    one, every request another number, so that the batch thins out step by step."""
    rng = random.Random(seed)
    prompt = [1, 64, 65] + [rng.randrange(2, 91) for _ in range(n - 3)]
    tails = [longest_tail] + [rng.randrange(2, longest_tail) for _ in range(n - 1)]
    rng.shuffle(prompt)
    reqs = {f"q{i}": [rng.randrange(vocab) for _ in range(p + t)] for i, (p, t) in enumerate(zip(prompt, tails))}
    return reqs, {f"q{i}": p for i, p in enumerate(prompt)}


def worst(got, want):
    """(error, request, position) of the worst position, relative to the request's largest logit."""
    out = (0.0, None, -1)
    for rid, w in want.items():
        per = np.max(np.abs(got[rid] - w), axis=1) / np.max(np.abs(w))
        i = int(np.argmax(per))
        if per[i] > out[0]:
            out = (float(per[i]), rid, i)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n", [("A", 8), ("E", 17), ("A", 33), ("D", 64)])
def test_large_batches_thin_out_through_the_step_function(model_folders, name, n, dtype):
    """n requests start together and go on one token per step for up to 72 steps; the batch shrinks from n rows to
    one, through every recorded row count.  Then a second batch of other requests runs in the slots and pages the
    first gave back."""
    folder = model_folders[name]
    vocab = TINY[name]["cfg"].vocab_size
    pm = PlainModel(folder)
    eng = engine_for(folder, dtype, max_tokens=64 * 3 * n, max_slots=n)
    for seed in (31, 32):
        reqs, prompt_len = unequal_requests(vocab, n, seed, 72)
        want = {rid: pm.logits(t).numpy() for rid, t in reqs.items()}
        got = run_trace(eng, batched_trace(reqs, [list(reqs)], prompt_len))
        err, rid, pos = worst(got, want)
        assert err <= TOL[dtype], f"batch of seed {seed}: {rid} position {pos} (prompt {prompt_len[rid]}) error {err:.3e}"
        assert eng.cache.tokens_held() == 0


def run_in_session(eng, reqs, prompt_len):
    """The requests' prompts in one step, then one decode session for all of them, fed from the requests' own
    tokens; rows whose tokens run out are parked while the others go on.  Logits of every position."""
    from exl3_server_b200 import StepEntry
    order = list(reqs)
    slots = {rid: eng.open() for rid in order}
    got = {rid: [None] * len(reqs[rid]) for rid in order}
    out = eng.step([StepEntry(slots[rid], reqs[rid][:prompt_len[rid]], "all") for rid in order]).float().cpu().numpy()
    row = 0
    for rid in order:
        for p in range(prompt_len[rid]):
            got[rid][p] = out[row]
            row += 1
    fed = dict(prompt_len)
    rows = list(order)
    session = eng.decode_session([slots[rid] for rid in order], max_new=max(len(t) for t in reqs.values()))
    while any(r is not None for r in rows):
        logits = session.step([reqs[rid][fed[rid]] if rid is not None else 0 for rid in rows]).float().cpu().numpy()
        ended = []
        for r, rid in enumerate(rows):
            if rid is None:
                continue
            got[rid][fed[rid]] = logits[r]
            fed[rid] += 1
            if fed[rid] >= len(reqs[rid]):
                ended.append(r)
        if ended:
            session.park(ended)
            for r in ended:
                eng.close(slots.pop(rows[r]))
                rows[r] = None
    session.close()
    eng.cache.check()
    return {rid: np.stack(rows_) for rid, rows_ in got.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n", [("E", 8), ("A", 17), ("D", 33), ("A", 64)])
def test_large_batches_thin_out_in_a_decode_session(model_folders, name, n, dtype):
    """The same through a decode session, as generation drives it: rows that ended become padding (``park``) and
    the graph of the full row count keeps running.  Two batches on one engine."""
    folder = model_folders[name]
    vocab = TINY[name]["cfg"].vocab_size
    pm = PlainModel(folder)
    eng = engine_for(folder, dtype, max_tokens=64 * 3 * n, max_slots=n)
    for seed in (41, 42):
        reqs, prompt_len = unequal_requests(vocab, n, seed, 72)
        want = {rid: pm.logits(t).numpy() for rid, t in reqs.items()}
        got = run_in_session(eng, reqs, prompt_len)
        err, rid, pos = worst(got, want)
        assert err <= TOL[dtype], f"batch of seed {seed}: {rid} position {pos} (prompt {prompt_len[rid]}) error {err:.3e}"
        assert eng.cache.tokens_held() == 0


def long_folder(name, tmp_path, positions=8192):
    from exl3_server_b200 import write_random_model
    t = TINY[name]
    cfg = dataclasses.replace(t["cfg"], max_position_embeddings=positions)
    return write_random_model(cfg, str(tmp_path / f"long{name}"), seed=77, std=0.08, norm_std=t["norm_std"],
                              dtype=torch.bfloat16, with_optional=t["biases"])


@pytest.mark.parametrize("name,dtype", [("D", "float32"), ("D", "bfloat16"), ("E", "bfloat16")])
def test_decoding_beyond_4096_tokens(name, dtype, tmp_path):
    """A prompt of 4,000 tokens, then 200 tokens one by one: the recorded step's context bucket changes at 4,096,
    the attention's chunks are at their longest, and page tables are wider than 64 pages."""
    folder = long_folder(name, tmp_path)
    toks = random_requests(TINY[name]["cfg"].vocab_size, [4200], seed=8)["r0"]
    want = PlainModel(folder).logits(toks).numpy()
    eng = engine_for(folder, dtype, max_tokens=4288)
    from exl3_server_b200 import StepEntry
    s = eng.open()
    head = eng.step([StepEntry(s, toks[:4000], [0, 1999, 3999])]).float().cpu().numpy()
    assert rel_err(head, want[[0, 1999, 3999]]) <= TOL[dtype]
    session = eng.decode_session([s], max_new=300)
    for p in range(4000, 4200):
        got = session.step([toks[p]]).float().cpu().numpy()
        err = rel_err(got, want[p:p + 1])
        assert err <= TOL[dtype], f"position {p}: error {err:.3e}"
    session.close()
    assert eng.length(s) == 4200
    eng.close(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "A"])
def test_rewinding_a_sequence_and_feeding_other_tokens(model_folders, name, dtype):
    """200 tokens, then back to a page's edge (128), to the middle of a page (100) and to nothing, each time
    followed by other tokens, as a piece and one by one: what was forgotten must not show."""
    from exl3_server_b200 import StepEntry
    from exl3_server_b200.cache import CacheError
    folder = model_folders[name]
    vocab = TINY[name]["cfg"].vocab_size
    first = random_requests(vocab, [200], seed=51)["r0"]
    pm = PlainModel(folder)
    eng = engine_for(folder, dtype, max_tokens=512)
    s = eng.open()
    eng.step([StepEntry(s, first, None)])
    held = eng.cache.tokens_held()
    for keep, seed in ((128, 52), (100, 53), (0, 54)):
        eng.truncate(s, keep)
        assert eng.length(s) == keep
        assert eng.cache.tokens_held() == (keep + 63) // 64 * 64 <= held
        other = random_requests(vocab, [40], seed=seed)["r0"]
        now = first[:keep] + other
        want = pm.logits(now).numpy()
        got = [eng.step([StepEntry(s, other[:30], "all")]).float().cpu().numpy()]
        for t in other[30:]:
            got.append(eng.step([StepEntry(s, [t], "last")]).float().cpu().numpy())
        err = rel_err(np.concatenate(got), want[keep:])
        assert err <= TOL[dtype], f"after rewinding to {keep}: error {err:.3e}"
        first = now
    with pytest.raises(CacheError, match="cannot truncate"):
        eng.truncate(s, eng.length(s) + 1)
    eng.close(s)
    assert eng.cache.tokens_held() == 0
    eng.cache.check()


def test_a_window_that_gave_pages_back_cannot_be_rewound(model_folders):
    from exl3_server_b200 import StepEntry
    from exl3_server_b200.cache import CacheError
    eng = engine_for(model_folders["D"], "bfloat16", max_tokens=512)     # a window of 80 keys on the last layer
    s = eng.open()
    eng.step([StepEntry(s, list(range(1, 301)), None)])
    with pytest.raises(CacheError, match="gave back pages"):
        eng.truncate(s, 100)
    eng.truncate(s, 290)                                              # inside what the window still holds
    assert eng.length(s) == 290
    eng.close(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_between_a_sessions_steps_does_not_disturb_it(model_folders, dtype):
    """A decode session of two rows is open; one-token steps of two other sequences (the same row count and
    page-table width) run between its steps.  Each user of the step function has buffers of its own."""
    from exl3_server_b200 import StepEntry
    folder = model_folders["B"]
    vocab = TINY["B"]["cfg"].vocab_size
    reqs = random_requests(vocab, [30, 45, 50, 20], seed=61)
    pm = PlainModel(folder)
    want = {rid: pm.logits(t).numpy() for rid, t in reqs.items()}
    eng = engine_for(folder, dtype)
    slots = {rid: eng.open() for rid in reqs}
    eng.step([StepEntry(slots[rid], reqs[rid][:10], None) for rid in reqs])
    session = eng.decode_session([slots["r0"], slots["r1"]], max_new=40)
    for p in range(10, 20):
        a = session.step([reqs["r0"][p], reqs["r1"][p]]).float().cpu().numpy()
        b = eng.step([StepEntry(slots["r2"], [reqs["r2"][p]], "last"),
                      StepEntry(slots["r3"], [reqs["r3"][p]], "last")]).float().cpu().numpy()
        assert rel_err(a, np.stack([want["r0"][p], want["r1"][p]])) <= TOL[dtype], f"session at position {p}"
        assert rel_err(b, np.stack([want["r2"][p], want["r3"][p]])) <= TOL[dtype], f"step at position {p}"
    # tokens that stay on the device: the session feeds its own argmax while the other two go on
    session.step([reqs["r0"][20], reqs["r1"][20]])
    ids = session.next_ids.tolist()
    eng.step([StepEntry(slots["r2"], [reqs["r2"][10]], None), StepEntry(slots["r3"], [reqs["r3"][10]], None)])
    after = session.step(None).float().cpu().numpy()
    for r, rid in enumerate(("r0", "r1")):
        ref = pm.logits(reqs[rid][:21] + [ids[r]]).numpy()[-1]
        assert rel_err(after[r:r + 1], ref[None]) <= TOL[dtype], rid
    session.close()
    runners = [r for pool in eng.decode_runners.values() for r in pool]
    assert len(runners) == 2 and all(r.holder is None for r in runners)
    for s in slots.values():
        eng.close(s)


def test_a_recorded_step_runs_again_after_a_later_one_needed_more_scratch(tmp_path):
    """One runner records a step per context bucket and the buckets need different amounts of scratch memory.
    The step recorded first (contexts up to 1,024 tokens) must still be right after steps for 2,048 and 3,072
    tokens were recorded, whatever has been allocated since."""
    from exl3_server_b200 import StepEntry
    folder = long_folder("E", tmp_path)                               # grouped heads of 128
    vocab = TINY["E"]["cfg"].vocab_size
    pm = PlainModel(folder)
    eng = engine_for(folder, "bfloat16", max_tokens=4096)

    def decode(tokens, start, steps, max_new):
        s = eng.open()
        eng.step([StepEntry(s, tokens[:start], None)])
        session = eng.decode_session([s], max_new=max_new)
        runner = session.runner
        got = np.concatenate([session.step([tokens[p]]).float().cpu().numpy() for p in range(start, start + steps)])
        session.close()
        eng.close(s)
        return got, runner

    short = random_requests(vocab, [110], seed=71)["r0"]
    long_one = random_requests(vocab, [2060], seed=72)["r0"]
    want = pm.logits(short).numpy()[100:110]
    got, runner = decode(short, 100, 10, 3990)
    assert rel_err(got, want) <= TOL["bfloat16"]
    _, again = decode(long_one, 2040, 20, 2050)                       # buckets 2,048 and 3,072 on the same runner
    assert again is runner and set(runner.graphs) == {1024, 2048, 3072}
    junk = [torch.full((1 << 16,), 3.0e4, device="cuda:0") for _ in range(64)]     # fills what may have been freed
    got, again = decode(short, 100, 10, 3990)
    assert again is runner
    assert rel_err(got, want) <= TOL["bfloat16"]
    del junk
    eng.check_kernels()


@pytest.mark.parametrize("head_dim,heads,kv_heads,short_form", [(64, 4, 2, 1), (128, 8, 1, 2), (128, 32, 2, 2)])
def test_every_way_of_merging_the_decode_attentions_chunks_is_reached_through_the_engine(head_dim, heads, kv_heads,
                                                                                          short_form, tmp_path,
                                                                                          monkeypatch):
    """One sequence of 1,500 tokens decodes in a cluster of two blocks per item and one of 200 in a block per item
    (with 8 query heads on one kv head of 128: eight groups of one head, in clusters again): the engine's own
    choice on a GPU of 148 SMs, recorded here; 40 sequences of 300 tokens in whatever way it picks: with 16 query
    heads on a kv head, two groups of 8 in one block, their warps walking the same pages.  Every position's logits against the plain implementation."""
    from exl3_server_b200 import LlamaConfig, write_random_model
    from exl3_server_b200.ops import kernels as K
    cfg = LlamaConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=heads, num_key_value_heads=kv_heads,
                      head_dim=head_dim, intermediate_size=176, vocab_size=301, rms_norm_eps=1e-5, rope_theta=10000.0,
                      max_position_embeddings=4096, tie_word_embeddings=False)
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=31, std=0.08, norm_std=0.1, dtype=torch.bfloat16)
    pm = PlainModel(folder)
    seen, twins = [], []
    real = K.attn_decode

    def spy(*args, **kw):
        seen.append(int(kw.get("in_block", 0)))
        twins.append(int(kw.get("twins", 1)))
        return real(*args, **kw)
    monkeypatch.setattr(K, "attn_decode", spy)
    eng = engine_for(folder, "bfloat16", max_tokens=40 * 320 + 2048)
    for n, prompt, tail, form in ((1, 1500, 24, 2), (1, 200, 24, short_form), (40, 300, 4, None)):
        seen.clear()
        twins.clear()
        reqs = random_requests(cfg.vocab_size, [prompt + tail] * n, seed=prompt)
        got = run_trace(eng, batched_trace(reqs, [list(reqs)], {r: prompt for r in reqs}))
        assert seen and (form is None or K.sm_count(torch.device("cuda:0")) != 148 or form in seen), \
            f"{n} x {prompt}: forms {sorted(set(seen))}"
        if n == 40 and heads // kv_heads == 16 and K.sm_count(torch.device("cuda:0")) == 148:
            assert 2 in twins
        for rid in list(reqs)[:3]:
            assert rel_err(got[rid], pm.logits(reqs[rid]).numpy()) <= TOL["bfloat16"], (n, prompt, rid)
        assert eng.cache.tokens_held() == 0
