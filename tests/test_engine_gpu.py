"""Engine-level behaviour on the GPU: long decoding, the first tokens of a
sequence, padding, slot reuse, windows' edges, generation through the entry
points, trace replay as a program, and errors that must come before any kernel."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, random_requests, rel_err, run_trace, tail_trace, whole_trace
from plain_llama import PlainModel

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine_for(folder, dtype, max_tokens=2048):
    from exl3_server_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D", "E"])
def test_long_decoding(model_folders, name, dtype):
    """A 40-token prompt, then 1100 tokens one by one: across page boundaries
    (64), attention chunk boundaries (256), the decode graph's context bucket
    (1024) and, in C and D, far past the window."""
    folder = model_folders[name]
    toks = random_requests(TINY[name]["cfg"].vocab_size, [1140], seed=5)["r0"]
    want = PlainModel(folder).logits(toks).numpy()
    eng = engine_for(folder, dtype)
    got = run_trace(eng, tail_trace({"r0": toks}, tail=1100))["r0"]
    per_pos = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
    bad = np.nonzero(per_pos > TOL[dtype])[0]
    assert bad.size == 0, f"first wrong position {bad[0]} of 1140, error {per_pos[bad[0]]:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_first_tokens_of_a_sequence(model_folders, name, dtype):
    """Positions 0, 1, 2 fed one by one, as a one-token prompt, and as a prompt."""
    folder = model_folders[name]
    toks = random_requests(TINY[name]["cfg"].vocab_size, [3], seed=9)["r0"]
    want = PlainModel(folder).logits(toks).numpy()
    eng = engine_for(folder, dtype)
    one_by_one = run_trace(eng, tail_trace({"r0": toks}, tail=3))["r0"]
    whole = run_trace(eng, whole_trace({"r0": toks}))["r0"]
    prompt1 = run_trace(eng, whole_trace({"r0": toks[:1]}))["r0"]
    for got in (one_by_one, whole):
        assert rel_err(got, want) <= TOL[dtype]
    assert rel_err(prompt1, want[:1]) <= TOL[dtype]


@pytest.mark.parametrize("name", ["A", "C"])
def test_padding_and_batch_mates_change_nothing_in_float32(model_folders, name):
    """Three sequences decode together (the decode graph pads them to four
    rows); each must get bit for bit what it gets alone."""
    from exl3_server_b200 import StepEntry
    folder = model_folders[name]
    reqs = random_requests(TINY[name]["cfg"].vocab_size, [70, 9, 33], seed=3)
    eng = engine_for(folder, "float32")
    alone = {}
    for rid, t in reqs.items():
        s = eng.open()
        eng.step([StepEntry(s, t[:-2], None)])
        a = eng.step([StepEntry(s, [t[-2]], "last")]).cpu()
        b = eng.step([StepEntry(s, [t[-1]], "last")]).cpu()
        alone[rid] = torch.cat([a, b])
        eng.close(s)
    slots = {rid: eng.open() for rid in reqs}
    eng.step([StepEntry(slots[rid], t[:-2], None) for rid, t in reqs.items()])
    a = eng.step([StepEntry(slots[rid], [t[-2]], "last") for rid, t in reqs.items()]).cpu()
    b = eng.step([StepEntry(slots[rid], [t[-1]], "last") for rid, t in reqs.items()]).cpu()
    for i, rid in enumerate(reqs):
        assert torch.equal(torch.stack([a[i], b[i]]), alone[rid]), rid
    for s in slots.values():
        eng.close(s)
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_reused_slot_shows_nothing_of_its_former_owner(model_folders, dtype):
    """A long sequence fills pages with large values and leaves; a short one
    gets the same slot and pages and must match the plain implementation."""
    from exl3_server_b200 import StepEntry
    folder = model_folders["B"]
    vocab = TINY["B"]["cfg"].vocab_size
    long_one = random_requests(vocab, [500], seed=1)["r0"]
    short = random_requests(vocab, [70], seed=2)["r0"]
    want = PlainModel(folder).logits(short).numpy()
    eng = engine_for(folder, dtype, max_tokens=512)
    s = eng.open()
    eng.step([StepEntry(s, long_one, None)])
    for g in eng.cache.groups:                        # make stale cache contents loud
        g.k.mul_(1000.0)
        g.v.mul_(1000.0)
    eng.close(s)
    s2 = eng.open()
    assert s2 == s
    got = eng.step([StepEntry(s2, short, "all")]).float().cpu().numpy()
    assert rel_err(got, want) <= TOL[dtype]
    got1 = eng.step([StepEntry(s2, [short[0]], "last")])     # and one more token through the decode path
    assert torch.isfinite(got1).all()
    eng.close(s2)


def test_window_edge_in_the_engine(model_folders):
    """Config D's last layer sees 80 keys.  Positions 76..89, where the window
    starts to cut keys off, are fed one by one and compared with the plain
    implementation; the plain implementation with a window of 79 instead of 80
    must give visibly other logits, so the comparison can tell the edge."""
    folder = model_folders["D"]
    vocab = TINY["D"]["cfg"].vocab_size
    toks = random_requests(vocab, [200], seed=21)["r0"]
    pm = PlainModel(folder)
    want = pm.logits(toks).numpy()
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(folder, dtype)
        # positions 79, 80, 81 are where the window starts to cut keys off; feed them one by one
        got = run_trace(eng, tail_trace({"r0": toks}, tail=200 - 76))["r0"]
        assert rel_err(got[76:90], want[76:90]) <= TOL[dtype]
        assert rel_err(got, want) <= TOL[dtype]
    # the plain implementation itself: a window of 79 or 81 gives other logits at position 120
    pm.c["windows"] = [0, 79]
    assert rel_err(pm.logits(toks).numpy()[120:121], want[120:121]) > 1e-4


@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_greedy_generation_through_the_entry_point(model_folders, name):
    from exl3_server_b200 import Engine, GenerateOptions
    folder = model_folders[name]
    cfg = TINY[name]["cfg"]
    pm = PlainModel(folder)
    prompts = list(random_requests(cfg.vocab_size, [5, 9, 13, 1, 66], seed=13).values())
    n = 12
    want = [pm.greedy(p, n) for p in prompts]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=2048)
    res = eng.generate(prompts, GenerateOptions(max_tokens=n, ignore_eos=True, max_batch=3))   # two batches
    assert [r.tokens for r in res] == want
    assert all(r.finish_reason == "length" and r.completion_tokens == n for r in res)
    assert eng.cache.tokens_held() == 0
    # bfloat16: the same tokens wherever the plain implementation's choice is clear
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=2048)
    res = eng.generate(prompts, GenerateOptions(max_tokens=n, ignore_eos=True))
    for p, r, w in zip(prompts, res, want):
        ids = list(p)
        for got, exp in zip(r.tokens, w):
            lg = pm.logits(ids)[-1]
            top2 = torch.topk(lg, 2).values
            clear = float(top2[0] - top2[1]) > 4 * TOL["bfloat16"] * float(lg.abs().max())
            if got != exp:
                assert not clear, f"bfloat16 picked {got}, plain picked {exp} with a clear margin"
                break
            ids.append(got)


def test_stop_tokens_and_early_ends(model_folders):
    from exl3_server_b200 import Engine, GenerateOptions
    folder = model_folders["A"]
    pm = PlainModel(folder)
    prompts = list(random_requests(256, [7, 11, 20], seed=17).values())
    free_run = [pm.greedy(p, 10) for p in prompts]
    stop = free_run[1][3]                                  # request 1 stops at its 4th token (or earlier)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024)
    res = eng.generate(prompts, GenerateOptions(max_tokens=10, stop_token_ids=[stop]))
    for r, w in zip(res, free_run):
        if stop in w:
            cut = w.index(stop) + 1
            assert r.tokens == w[:cut] and r.finish_reason == "stop"
        else:
            assert r.tokens == w and r.finish_reason == "length"
    assert res[1].finish_reason == "stop" and len(res[1].tokens) <= 4


def test_temperature_sampling_is_seeded(model_folders):
    from exl3_server_b200 import Engine, GenerateOptions, SampleOptions
    eng = Engine.from_folder(model_folders["B"], dtype="bfloat16", max_tokens=1024)
    prompts = [[1, 2, 3], [4, 5, 6, 7]]
    for so in (SampleOptions(temperature=0.9, seed=5), SampleOptions(temperature=0.9, seed=5, top_k=20, top_p=0.9)):
        opt = GenerateOptions(max_tokens=12, ignore_eos=True, sample=so)
        a = eng.generate(prompts, opt)
        b = eng.generate(prompts, opt)
        assert [r.tokens for r in a] == [r.tokens for r in b]
    other = eng.generate(prompts, GenerateOptions(max_tokens=12, ignore_eos=True,
                                                  sample=SampleOptions(temperature=0.9, seed=6)))
    assert [r.tokens for r in other] != [r.tokens for r in a]


def test_sampled_generation_is_the_same_one_step_ahead_of_the_host(model_folders):
    """Sampled tokens feed the next step on the device; the host reads them a step later.  Requests of unequal
    lengths that end on a stop token at different times: the same tokens as with the host in every step."""
    from exl3_server_b200 import Engine, GenerateOptions, SampleOptions
    eng = Engine.from_folder(model_folders["D"], dtype="bfloat16", max_tokens=2048)
    prompts = [[1, 2, 3], [4, 5, 6, 7, 8, 9], [10], [11, 12]]
    so = SampleOptions(temperature=0.9, top_k=50, top_p=0.95, repetition_penalty=1.15, frequency_penalty=0.05, seed=21)
    runs = []
    for ahead in (True, False):
        opt = GenerateOptions(max_tokens=40, stop_token_ids=[17, 33, 52, 80, 101], sample=so, run_ahead=ahead)
        runs.append(eng.generate(prompts, opt))
        assert eng.cache.tokens_held() == 0
    assert [r.tokens for r in runs[0]] == [r.tokens for r in runs[1]]
    assert [r.finish_reason for r in runs[0]] == [r.finish_reason for r in runs[1]]
    assert len({len(r.tokens) for r in runs[0]}) > 1 or all(r.finish_reason == "length" for r in runs[0])


def test_sampling_on_the_device_follows_the_host_sampler():
    """The same requests sampled from logits on the device and from a copy on the host: filters, penalties over
    the growing context, a greedy row among them, every request with its own generator."""
    from exl3_server_b200.sampling import SampleOptions
    from exl3_server_b200.sampling.sampler import RowSampler, sample_rows
    opts = [SampleOptions(temperature=0.8, top_k=30, top_p=0.9, seed=3),
            SampleOptions(temperature=1.2, min_p=0.03, repetition_penalty=1.2, presence_penalty=0.3,
                          frequency_penalty=0.1, seed=4),
            SampleOptions(temperature=0.0, repetition_penalty=1.5),
            SampleOptions(temperature=1.0, seed=5)]
    prompts = [[5, 6, 7], [8, 8, 8, 9], [1], [2, 3]]
    V = 4000
    g = torch.Generator().manual_seed(17)
    dev_rows = [RowSampler(o, i, p) for i, (o, p) in enumerate(zip(opts, prompts))]
    host_rows = [RowSampler(o, i, p) for i, (o, p) in enumerate(zip(opts, prompts))]
    for _ in range(40):
        logits = 3.0 * torch.randn(len(opts), V, generator=g)
        on_device = sample_rows(logits.to("cuda:0"), dev_rows)
        on_host = sample_rows(logits, host_rows)
        assert on_device == on_host
    assert [r.context for r in dev_rows] == [r.context for r in host_rows]


def test_errors_come_before_any_kernel(model_folders):
    from exl3_server_b200 import Engine, StepEntry, StepError
    from exl3_server_b200.cache import CacheFull
    eng = Engine.from_folder(model_folders["A"], dtype="float32", max_tokens=128)
    s = eng.open()
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([StepEntry(s, [1, 256])])
    with pytest.raises(StepError, match="twice"):
        eng.step([StepEntry(s, [1]), StepEntry(s, [2])])
    with pytest.raises(StepError, match="at least one token"):
        eng.step([StepEntry(s, [])])
    with pytest.raises(StepError, match="not live"):
        eng.step([StepEntry(s + 1, [1])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(StepError, match="max_position_embeddings"):
        eng.step([StepEntry(s, [1] * 513)])
    with pytest.raises(CacheFull):
        eng.step([StepEntry(s, [1] * 129)])
    assert eng.length(s) == 0 and eng.steps_run == 0
    eng.step([StepEntry(s, [1, 2, 3])])
    assert eng.length(s) == 3
    eng.close(s)


def test_no_cpu_path():
    from exl3_server_b200 import Engine
    from exl3_server_b200.engine.engine import load_model
    from exl3_server_b200.ops.lib import KernelLibraryError
    import tempfile
    from helpers import make_folder
    with tempfile.TemporaryDirectory() as d:
        make_folder("A", d)
        model = load_model(d, "float32", "cpu")
        with pytest.raises(KernelLibraryError, match="CUDA device only"):
            Engine(model, max_tokens=128)


def test_trace_run_as_a_program(model_folders, tmp_path):
    """bin/trace_run on its own: JSON steps on stdin, <step>.f32 files out, one
    'done' line per step; its numbers equal the in-process replay's."""
    folder = model_folders["C"]
    reqs = random_requests(TINY["C"]["cfg"].vocab_size, [40, 7], seed=4)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": reqs["r0"][:38], "want": [0, 37]},
                                {"id": "b", "tokens": reqs["r1"][:6], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [reqs["r0"][38]], "want": [0]},
                                {"id": "b", "tokens": [reqs["r1"][6]], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [reqs["r0"][39]], "want": []}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "b", "tokens": reqs["r1"], "want": [6]}], "end": ["b"]},
    ]
    pm = PlainModel(folder)
    la, lb = pm.logits(reqs["r0"]).numpy(), pm.logits(reqs["r1"]).numpy()
    vocab = TINY["C"]["cfg"].vocab_size
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                           timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert p.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
        assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "3.f32"]          # step 2 wanted nothing
        s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, vocab)
        s1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, vocab)
        s3 = np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, vocab)
        assert s0.shape[0] == 2 and s1.shape[0] == 2 and s3.shape[0] == 1
        assert rel_err(s0, la[[0, 37]]) <= TOL[dtype]
        assert rel_err(s1, np.stack([la[38], lb[6]])) <= TOL[dtype]
        assert rel_err(s3, lb[6:7]) <= TOL[dtype]


def test_command_line(model_folders):
    from exl3_server_b200 import Engine, GenerateOptions
    folder = model_folders["B"]
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024)
    want = eng.generate([[5, 6, 7], [9]], GenerateOptions(max_tokens=6, ignore_eos=True))
    p = subprocess.run([sys.executable, "-m", "exl3_server_b200", "--model", folder, "-p", "5,6,7", "--prompt=9",
                        "--max-tokens", "6", "--ignore-eos", "--temp=0"], capture_output=True, text=True, cwd=ROOT,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.strip().splitlines() if l]
    assert lines == [",".join(map(str, r.tokens)) for r in want]
    assert "3 prompt + 6 generated tokens" in p.stderr and "tok/s | length]" in p.stderr
    bad = subprocess.run([sys.executable, "-m", "exl3_server_b200", "--model", folder, "--serve"], capture_output=True,
                         text=True, cwd=ROOT, timeout=120)
    assert bad.returncode == 2


def test_kernels_report_no_bounded_wait_that_ran_out(model_folders):
    """After real work through the tensor-core kernels (heads of 64) no kernel has given up on a wait."""
    from exl3_server_b200 import Engine, GenerateOptions
    eng = Engine.from_folder(model_folders["D"], dtype="bfloat16", max_tokens=1024)
    toks = random_requests(TINY["D"]["cfg"].vocab_size, [300, 70], seed=2)
    res = eng.generate(list(toks.values()), GenerateOptions(max_tokens=8, ignore_eos=True))
    assert all(r.completion_tokens == 8 for r in res)
    eng.check_kernels()


def test_stats_count_what_the_steps_had_to_do(model_folders):
    """Tokens, steps, bytes and flops of a prompt step, three one-token steps and a generation call, against the
    sizes of configuration B worked out by hand."""
    from exl3_server_b200 import Engine, GenerateOptions, StepEntry
    cfg = TINY["B"]["cfg"]
    eng = Engine.from_folder(model_folders["B"], dtype="bfloat16", max_tokens=1024)
    H, I, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    layer = (q + 2 * kv) * H + H * q + 3 * I * H                       # matrix weights of a layer
    norms = (2 * L + 1) * H
    assert eng.model.weight_bytes() == 2 * (L * layer + norms + V * H)   # the untied head's matrix; the embedding is not read
    s = eng.open()
    eng.step([StepEntry(s, list(range(1, 41)), "last")])
    for t in (5, 6, 7):
        eng.step([StepEntry(s, [t], "last")])
    st = eng.stats
    assert (st.steps, st.prompt_steps, st.decode_steps, st.tokens) == (4, 1, 3, 43)
    assert st.weight_bytes == 4 * eng.model.weight_bytes()
    per_token = 2 * L * 2 * kv                                          # bfloat16 keys and values of every layer
    assert st.cache_bytes == per_token * (40 + 41 + 42 + 43)
    keys = 40 * 41 // 2 + 41 + 42 + 43
    want = 2.0 * (L * layer + norms) * 43 + 2.0 * V * H * 4 + 4.0 * L * q * keys
    assert abs(st.flops - want) <= 1e-9 * want
    eng.close(s)
    eng.generate([[1, 2, 3], [4, 5]], GenerateOptions(max_tokens=5, ignore_eos=True))
    g = eng.last_generate_stats
    assert g.prompt_steps == 1 and g.decode_steps == 4 and g.tokens == 5 + 2 * 4
    eng.check_kernels()                                                 # the cache's guard words among other things
