"""The engine against the plain implementation at layer sizes of real models (two layers of each, random
weights): the benchmark's MiniCPM-2B sizes (36 heads of 64, width 2304, vocabulary 122753, tied head) and
Llama-3-8B-like sizes (32 query heads on 8 key/value heads of 128, width 4096, feed-forward 14336, vocabulary
128256).  The tiny configurations of the other tests reach every option; these reach the shapes the kernels are
tuned for: whole prompt, then the last 40 tokens one by one."""
import os
import sys

import numpy as np
import pytest
import torch

from helpers import TOL, run_trace, tail_trace, whole_trace
from plain_llama import PlainModel

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _configs():
    import bench
    from exl3_server_b200 import LlamaConfig
    return {
        "minicpm-2b": LlamaConfig(**{**bench.BENCH_MODEL, "num_hidden_layers": 2}),
        "llama-8b-like": LlamaConfig(**{**bench.OTHER_SIZES["llama-8b-like"][0], "num_hidden_layers": 2}),
    }


@pytest.mark.parametrize("name", ["minicpm-2b", "llama-8b-like"])
def test_two_layers_of_real_sizes(tmp_path, name):
    from exl3_server_b200 import Engine, write_random_model
    cfg = _configs()[name]
    folder = str(tmp_path / name)
    write_random_model(cfg, folder, seed=3, std=0.02)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg.vocab_size, (200,), generator=g).tolist()
    want = PlainModel(folder).logits(toks).numpy()
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
        for what, trace in (("whole", whole_trace({"r0": toks})), ("last 40 one by one", tail_trace({"r0": toks}, tail=40))):
            got = run_trace(eng, trace)["r0"]
            per_pos = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
            bad = np.nonzero(per_pos > TOL[dtype])[0]
            assert bad.size == 0, f"{name} {dtype} {what}: first wrong position {bad[0]}, error {per_pos[bad[0]]:.3e}"
        del eng
        torch.cuda.empty_cache()
