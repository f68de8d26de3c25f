"""What can be anchored on the reference's own code: its sampler and its safetensors reader compile without
Apple's MLX.  ``tests/golden/reference_golden.json`` holds what they answered to the cases of
``tests/golden/make_reference_golden.py`` (compiled from the reference's files, which are not kept here).  The
host sampler must pick the same tokens draw for draw; the container this library writes must read back here as
the reference's reader saw it.  The forward pass has no such anchor: src/model.cpp needs MLX."""
import hashlib
import importlib.util
import json
import os
import shutil

import numpy as np
import pytest
import torch

from exl3_server_b200.sampling import SampleOptions, SplitMix64, sample_token
from exl3_server_b200.weights import TensorStore, write_safetensors

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_reference_golden", os.path.join(HERE, "golden", "make_reference_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)

with open(os.path.join(HERE, "golden", "reference_golden.json")) as f:
    GOLDEN = json.load(f)


@pytest.mark.parametrize("i", range(len(G.SAMPLER_CASES)))
def test_host_sampler_picks_the_reference_samplers_tokens(i):
    case = G.SAMPLER_CASES[i]
    want = [int(t) for t in GOLDEN["sampler"][i]["tokens"].split()]
    opt = SampleOptions(temperature=case["temperature"], top_p=case["top_p"], top_k=case["top_k"], min_p=case["min_p"],
                        repetition_penalty=case["rep"], presence_penalty=case["pres"], frequency_penalty=case["freq"],
                        seed=case["seed"])
    rng = SplitMix64(case["seed"])
    context = list(case["context"])
    got = []
    for d in range(case["draws"]):
        tok = sample_token(G.golden_logits(case["seed"] * 1000 + d, case["n"]), opt, context, rng)
        context.append(tok)
        got.append(tok)
    assert got == want
    if case["temperature"] > 0:
        assert len(set(got)) > 5                     # the draws are draws, not one token again and again


def test_the_container_reads_back_as_the_reference_reader_saw_it(tmp_path):
    path = str(tmp_path / "model.safetensors")
    tensors = G.container_tensors()
    write_safetensors(path, tensors.items(), metadata={"format": "pt"})
    with open(path, "rb") as f:
        assert hashlib.sha256(f.read()).hexdigest() == GOLDEN["container_sha256"], \
            "the writer's bytes changed: make the golden file again"
    names = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I32": torch.int32, "I16": torch.int16}
    store = TensorStore(str(tmp_path))
    lines = [l for l in GOLDEN["container"] if not l.startswith("wrong-type")]
    assert len(lines) == len(tensors) and GOLDEN["container"][-1] == "wrong-type access: refused"
    for line in lines:
        name, dtype, shape, nbytes, first, last = line.split()
        t = store.tensor(name)
        assert t.dtype == names[dtype] and list(t.shape) == json.loads(shape)
        assert t.numel() * t.element_size() == int(nbytes)
        assert torch.equal(t, tensors[name])
        raw = t.contiguous().view(torch.uint8).numpy().tobytes()
        w = t.element_size()
        assert int.from_bytes(raw[:w], "little") == int(first) and int.from_bytes(raw[-w:], "little") == int(last)


@pytest.mark.skipif(not os.path.isdir(os.path.join(G.DEFAULT_REFERENCE, "src")) or shutil.which("g++") is None,
                    reason="needs the reference's sources and g++")
def test_the_committed_golden_file_is_what_the_reference_answers_today():
    assert G.make(G.DEFAULT_REFERENCE) == GOLDEN
