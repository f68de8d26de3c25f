"""The generation loop's decisions, with a scripted engine (no GPU): batches
of unequal prompts, stop tokens, rows that end early, one batch after another,
cancellation, and what each request is charged."""
import pytest
import torch

from exl3_server_b200 import GenerateOptions, SampleOptions
from exl3_server_b200.engine.generate import generate, plan_batches

V = 16


class ScriptedEngine:
    """Next token = (last token + 1) mod V.  Records everything it is asked."""

    def __init__(self, cache_tokens=64 * 64, stop=(0,)):
        self.stop_token_ids = list(stop)
        self.cache_tokens = cache_tokens
        self.free = list(range(63, -1, -1))
        self.live = {}
        self.calls = []
        self.opened = []
        self.closed = []

    def open(self):
        s = self.free.pop()
        self.live[s] = []
        self.opened.append(s)
        return s

    def close(self, s):
        assert s in self.live, "slot closed twice"
        del self.live[s]
        self.free.append(s)
        self.closed.append(s)

    def _logits(self, slots):
        out = torch.full((len(slots), V), -1.0)
        for r, s in enumerate(slots):
            out[r, (self.live[s][-1] + 1) % V] = 1.0
        return out

    def step(self, entries):
        self.calls.append(("step", [(e.slot, len(e.tokens)) for e in entries]))
        for e in entries:
            self.live[e.slot].extend(e.tokens)
        return self._logits([e.slot for e in entries])

    def decode_session(self, slots, max_new=0):
        eng = self

        class Session:
            next_ids = None

            def step(self, tokens):
                eng.calls.append(("decode", list(slots)))
                for s, t in zip(slots, tokens):
                    eng.live[s].append(t)
                return eng._logits(slots)

            def close(self):
                pass

        return Session()


def test_unequal_prompts_stop_length_and_early_ends():
    eng = ScriptedEngine(stop=(0,))
    prompts = [[13], [5, 6, 7], [1, 2, 3, 4, 10, 11]]
    res = generate(eng, prompts, GenerateOptions(max_tokens=4))
    assert res[0].tokens == [14, 15, 0] and res[0].finish_reason == "stop"      # the stop token is kept
    assert res[1].tokens == [8, 9, 10, 11] and res[1].finish_reason == "length"
    assert res[2].tokens == [12, 13, 14, 15] and res[2].finish_reason == "length"
    assert [r.prompt_tokens for r in res] == [1, 3, 6]
    assert [r.completion_tokens for r in res] == [3, 4, 4]
    # one prefill step with all prompts, then one token per live row; no step after the last token
    assert eng.calls[0] == ("step", [(0, 1), (1, 3), (2, 6)])
    assert [len(c[1]) for c in eng.calls[1:]] == [3, 3, 2]
    assert not eng.live and sorted(eng.closed) == sorted(eng.opened)


def test_ignore_eos_and_custom_stop_ids():
    eng = ScriptedEngine(stop=(0,))
    res = generate(eng, [[14]], GenerateOptions(max_tokens=4, ignore_eos=True))
    assert res[0].tokens == [15, 0, 1, 2] and res[0].finish_reason == "length"
    res = generate(eng, [[14]], GenerateOptions(max_tokens=8, stop_token_ids=[2]))
    assert res[0].tokens == [15, 0, 1, 2] and res[0].finish_reason == "stop"


def test_batches_one_after_another_reuse_slots():
    eng = ScriptedEngine()
    prompts = [[i + 1] for i in range(5)]
    res = generate(eng, prompts, GenerateOptions(max_tokens=2, max_batch=2))
    assert [r.tokens for r in res] == [[2, 3], [3, 4], [4, 5], [5, 6], [6, 7]]
    prefills = [c for c in eng.calls if c[0] == "step"]
    assert [len(c[1]) for c in prefills] == [2, 2, 1]
    assert len(set(eng.opened)) == 2 and len(eng.opened) == 5      # two slots served five requests
    assert not eng.live


def test_empty_prompt_and_zero_budget():
    eng = ScriptedEngine()
    res = generate(eng, [[], [3]], GenerateOptions(max_tokens=2))
    assert res[0].finish_reason == "stop" and res[0].tokens == []      # src/engine.cpp:227-230
    assert res[1].tokens == [4, 5]
    res = generate(eng, [[3]], GenerateOptions(max_tokens=0))
    assert res[0].tokens == [] and res[0].finish_reason == "length" and not eng.calls[2:]


def test_cancel_frees_everything():
    eng = ScriptedEngine()
    polls = {"n": 0}

    def cancelled():
        polls["n"] += 1
        return polls["n"] > 2

    res = generate(eng, [[1], [2]], GenerateOptions(max_tokens=50), cancelled=cancelled)
    assert all(r.finish_reason == "cancelled" for r in res)
    assert [len(r.tokens) for r in res] == [2, 2]
    assert not eng.live


def test_on_token_streams_in_order():
    eng = ScriptedEngine()
    seen = []
    generate(eng, [[1], [7]], GenerateOptions(max_tokens=2), on_token=lambda i, t: seen.append((i, t)))
    assert seen == [(0, 2), (1, 8), (0, 3), (1, 9)]


def test_plan_batches_respects_the_cache():
    # each request may grow to prompt + 100 tokens, counted in pages of 64
    assert plan_batches([10, 10, 10], 100, max_batch=8, cache_tokens=256) == [[0, 1], [2]]
    assert plan_batches([10, 0, 10], 100, max_batch=1, cache_tokens=4096) == [[0], [2]]
    with pytest.raises(ValueError, match="do not fit"):
        plan_batches([1000], 100, 8, 512)


def test_seeded_temperature_is_reproducible():
    eng = ScriptedEngine()
    opt = GenerateOptions(max_tokens=6, ignore_eos=True, sample=SampleOptions(temperature=1.5, seed=42))
    a = generate(eng, [[1], [1]], opt)
    b = generate(eng, [[1], [1]], opt)
    assert [r.tokens for r in a] == [r.tokens for r in b]
    assert a[0].tokens != a[1].tokens                  # each request has a stream of its own (seed + index)


def test_plan_batches_refuses_more_positions_than_the_model_has():
    assert plan_batches([10, 20], 100, 8, 4096, max_positions=120) == [[0, 1]]
    with pytest.raises(ValueError, match="exceed max_position_embeddings 119"):
        plan_batches([10, 20], 100, 8, 4096, max_positions=119)


class AheadEngine(ScriptedEngine):
    """The scripted engine with a session that can run one step ahead of the host, as the real one does:
    ``step(None)`` feeds what the last step chose, ``fetch_ids`` hands those tokens out later, ``park`` turns
    rows into padding."""

    max_positions = 0

    def decode_session(self, slots, max_new=0):
        eng = self

        class Fetched:
            def __init__(self, ids):
                self.ids = ids

            def get(self):
                return list(self.ids)

        class Session:
            def __init__(self):
                self.rows = list(slots)
                self.chosen = None
                self.parked = []

            def step(self, tokens):
                live = [s for s in self.rows if s is not None]
                eng.calls.append(("decode", live))
                feed = tokens if tokens is not None else self.chosen
                for r, s in enumerate(self.rows):
                    if s is not None:
                        eng.live[s].append(feed[r])
                self.chosen = [(eng.live[s][-1] + 1) % V if s is not None else 0 for s in self.rows]
                return None

            def fetch_ids(self, ids=None):
                return Fetched(self.chosen)

            def park(self, rows):
                for r in rows:
                    assert self.rows[r] is not None, "row parked twice"
                    self.parked.append(r)
                    self.rows[r] = None

            def close(self):
                pass

        self.session = Session()
        return self.session


def test_run_ahead_spends_no_step_after_the_length_limit():
    eng = AheadEngine(stop=())
    res = generate(eng, [[1], [5, 6]], GenerateOptions(max_tokens=4))
    assert [r.tokens for r in res] == [[2, 3, 4, 5], [7, 8, 9, 10]]
    assert all(r.finish_reason == "length" for r in res)
    # the prompts' step gives token 1; tokens 2, 3 and 4 take one decode step each and nothing runs after them
    assert [c[0] for c in eng.calls] == ["step", "decode", "decode", "decode"]
    assert not eng.live


def test_run_ahead_parks_rows_that_stop_and_goes_on_with_the_rest():
    eng = AheadEngine(stop=(0,))
    res = generate(eng, [[13], [3]], GenerateOptions(max_tokens=6))
    assert res[0].tokens == [14, 15, 0] and res[0].finish_reason == "stop"
    assert res[1].tokens == [4, 5, 6, 7, 8, 9] and res[1].finish_reason == "length"
    assert eng.session.parked == [0]
    decodes = [c[1] for c in eng.calls if c[0] == "decode"]
    # the stop token was seen one step late: the row ran once more into its own pages, then only the other row
    assert [len(d) for d in decodes] == [2, 2, 2, 1, 1]
    assert not eng.live and sorted(eng.closed) == sorted(eng.opened)
