"""The generation loop above the step function.

Requests are run in batches, one batch after another, as many as there are
requests.  The prompts of a batch, of unequal lengths, go through the model in
one step; then every live request advances one token per step.  A request ends
on a stop token (which is kept in its tokens), at ``max_tokens`` or when the
caller cancels; its slot goes back to the cache at once and the others carry
on.  This is the reference's serial loop (src/engine.cpp:341-353, stop rules of
``Emitter::emit`` src/engine.cpp:103-109, reasons "stop" / "length" /
"cancelled" src/engine.h:63) made batched; unlike the reference no forward
pass is spent after a request's last token (src/engine.cpp:349-350).

The loop only needs an object with ``open()``, ``close(slot)`` and
``step(entries) -> logits`` and ``decode_session(slots, max_new)`` (an object
with ``step(tokens) -> logits``, ``next_ids`` and ``close()``); its decisions are
tested with a scripted one.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.options import SampleOptions
from ..sampling.sampler import RowSampler, launch_on_device, on_device, record, sample_rows
from ..cache.kv import PAGE_SIZE
from .engine import StepEntry


@dataclass
class GenerateOptions:
    sample: SampleOptions = field(default_factory=SampleOptions)
    max_tokens: int = 512                       # src/engine.h:50
    ignore_eos: bool = False
    stop_token_ids: Optional[Sequence[int]] = None   # None: the model's eos ids
    max_batch: int = 64                         # most requests that start together
    run_ahead: bool = True                      # launch step k + 1 before reading step k's tokens (sampling on the device)


@dataclass
class GenerateResult:
    tokens: List[int] = field(default_factory=list)   # generated ids, stop token included
    finish_reason: str = ""                            # "stop" | "length" | "cancelled"
    prompt_tokens: int = 0
    completion_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, max_batch: int, cache_tokens: int,
                 max_positions: int = 0, page: int = PAGE_SIZE) -> List[List[int]]:
    """Splits request indices, in order, into batches that fit the cache: a
    request may grow to its prompt plus ``max_tokens`` tokens, counted in whole
    pages.  With ``max_positions`` a request that could grow beyond the model's positions is refused here,
    before anything runs, as the step function would refuse it later."""
    def need(n: int) -> int:
        # one token more than asked for: greedy decoding runs one step ahead of the host
        return (n + max_tokens + 1 + page - 1) // page * page

    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if n == 0:
            continue                              # answered without a forward pass
        if max_positions and n + max_tokens > max_positions:
            raise ValueError(f"request {i}: {n + max_tokens} positions exceed max_position_embeddings {max_positions}")
        if need(n) > cache_tokens:
            raise ValueError(f"request {i}: {n} prompt + {max_tokens} new tokens do not fit a cache of "
                             f"{cache_tokens} tokens")
        if cur and (len(cur) >= max_batch or used + need(n) > cache_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need(n)
    if cur:
        batches.append(cur)
    return batches


def generate(engine, prompts: Sequence[Sequence[int]], options: Optional[GenerateOptions] = None,
             cancelled: Optional[Callable[[], bool]] = None,
             on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerateResult]:
    """Generates for every prompt (lists of token ids).  ``on_token(request,
    token)`` is called for each new token; ``cancelled()`` is polled once per
    step."""
    opt = options or GenerateOptions()
    if opt.max_tokens < 0 or opt.max_batch < 1:
        raise ValueError("max_tokens must be >= 0 and max_batch >= 1")
    stops = set(opt.stop_token_ids if opt.stop_token_ids is not None else engine.stop_token_ids)
    results = [GenerateResult(prompt_tokens=len(p)) for p in prompts]
    for i, p in enumerate(prompts):
        if len(p) == 0 or opt.max_tokens == 0:
            results[i].finish_reason = "stop" if len(p) == 0 else "length"   # src/engine.cpp:227-230
    todo = [len(p) if opt.max_tokens > 0 else 0 for p in prompts]
    for batch in plan_batches(todo, opt.max_tokens, opt.max_batch, engine.cache_tokens,
                              getattr(engine, "max_positions", 0), getattr(engine, "page_size", PAGE_SIZE)):
        _run_batch(engine, prompts, batch, results, opt, stops, cancelled, on_token)
        check = getattr(engine, "check_kernels", None)
        if check is not None:
            check()                                       # the batch's tokens are on the host: no extra wait
    return results


def _run_batch(engine, prompts, batch, results, opt, stops, cancelled, on_token) -> None:
    slots = {i: engine.open() for i in batch}
    samplers = {i: RowSampler(opt.sample, i, prompts[i]) for i in batch}
    state = {"d0": 0.0}

    def emit(i: int, tok: int) -> bool:
        """Records a token; True when the request has ended (its slot is freed at once)."""
        r = results[i]
        r.tokens.append(tok)
        r.completion_tokens += 1
        if on_token is not None:
            on_token(i, tok)
        if not opt.ignore_eos and tok in stops:
            r.finish_reason = "stop"
        elif r.completion_tokens >= opt.max_tokens:
            r.finish_reason = "length"
        if r.finish_reason:
            r.decode_seconds = time.perf_counter() - state["d0"]
            return True
        return False

    session = None
    live = list(batch)
    try:
        t0 = time.perf_counter()
        logits = engine.step([StepEntry(slots[i], prompts[i], "last") for i in live])
        if cancelled is not None and cancelled():              # polled before every sampling (src/engine.cpp:344)
            for i in live:
                results[i].finish_reason = "cancelled"
                results[i].prefill_seconds = time.perf_counter() - t0
            return
        picked = sample_rows(logits, [samplers[i] for i in live])
        pf = time.perf_counter() - t0              # the prefill ends when its logits have been used once
        for i in live:
            results[i].prefill_seconds = pf
        state["d0"] = time.perf_counter()
        nxt = []
        for i, tok in zip(live, picked):
            if emit(i, tok):
                engine.close(slots.pop(i))
            else:
                nxt.append((i, tok))
        live = [i for i, _ in nxt]
        if not live:
            return
        remaining = opt.max_tokens - min(results[i].completion_tokens for i in live)
        session = engine.decode_session([slots[i] for i in live], max_new=remaining + 1)
        greedy = all(samplers[i].opt.greedy and not samplers[i].opt.has_penalties for i in live)
        ahead = opt.run_ahead and hasattr(session, "fetch_ids")
        if greedy and ahead:
            _decode_ahead(engine, session, live, [t for _, t in nxt], slots, results, emit, cancelled, state,
                          opt.max_tokens)
        elif ahead and on_device(logits, [samplers[i] for i in live]):
            _decode_ahead(engine, session, live, [t for _, t in nxt], slots, results, emit, cancelled, state,
                          opt.max_tokens, samplers=[samplers[i] for i in live])
        else:
            session = _decode_in_step(engine, session, nxt, slots, samplers, results, opt, emit, cancelled, state)
    finally:
        if session is not None:
            session.close()
        for s in slots.values():
            engine.close(s)


def _decode_in_step(engine, session, nxt, slots, samplers, results, opt, emit, cancelled, state):
    """One step, then the host samples, then the next step.  Any sampler."""
    live = [i for i, _ in nxt]
    while live:
        if cancelled is not None and cancelled():
            for i in live:
                results[i].finish_reason = "cancelled"
                results[i].decode_seconds = time.perf_counter() - state["d0"]
            break
        logits = session.step([tok for _, tok in nxt])
        picked = sample_rows(logits, [samplers[i] for i in live], session.next_ids)
        nxt, retired = [], False
        for i, tok in zip(live, picked):
            if emit(i, tok):
                if session is not None:
                    session.close()
                    session = None
                engine.close(slots.pop(i))              # the slot is free for the next batch at once
                retired = True
            else:
                nxt.append((i, tok))
        live = [i for i, _ in nxt]
        if live and (session is None or retired):
            if session is not None:
                session.close()
            remaining = opt.max_tokens - min(results[i].completion_tokens for i in live)
            session = engine.decode_session([slots[i] for i in live], max_new=remaining + 1)
    return session


def _decode_ahead(engine, session, rows, first_tokens, slots, results, emit, cancelled, state, max_tokens,
                  samplers=None) -> None:
    """Decoding one step ahead of the host.  The tokens of a step (its argmax, or with ``samplers`` what the
    device sampler draws from its logits) feed the next step on the device, so step k + 1 is launched before
    the host has seen the tokens of step k; the host reads them (pinned copy) and decides who has ended while
    the GPU works.  A row that ended on a stop token has run one step too many into its own pages, is turned
    into padding, and its slot is freed.  When the tokens on their way are the last that ``max_tokens`` allows
    to every live row, no step is launched ahead of them: only an unforeseen stop token costs a step."""
    alive = [True] * len(rows)

    def launch(tokens):
        logits = session.step(tokens)
        if samplers is None:
            return session.fetch_ids()
        ids = launch_on_device(logits, samplers)         # rows that ended draw too; nobody reads their tokens
        session.feed(ids)
        return session.fetch_ids(ids)

    pending = launch(first_tokens)
    while True:
        if cancelled is not None and cancelled():
            for r, i in enumerate(rows):
                if alive[r]:
                    results[i].finish_reason = "cancelled"
                    results[i].decode_seconds = time.perf_counter() - state["d0"]
            return
        last = all(results[i].completion_tokens + 1 >= max_tokens for r, i in enumerate(rows) if alive[r])
        following = None if last else launch(None)    # launched before the pending tokens are looked at
        toks = pending.get()
        if samplers is not None:
            record(samplers, toks)
        ended = [r for r, i in enumerate(rows) if alive[r] and emit(i, toks[r])]
        for r in ended:
            alive[r] = False
        if ended and any(alive):
            session.park(ended)                       # the others go on; nothing to re-arrange when all have ended
        for r in ended:
            engine.close(slots.pop(rows[r]))
        if not any(alive):
            return
        pending = following
