"""Random tiny configurations (seeded): head sizes in steps of 16, any number of heads and groups (four of them
with 10 to 16 query heads per kv head and requests of up to 520 tokens), widths,
feed-forward sizes and vocabularies that are no power of two, windows on some layers, the scale constants on or
off, biases on or off.  Each is replayed whole, with the last 20 tokens one by one and in unequal batches, in
float32 and in bfloat16, against the plain implementation."""
import random

import numpy as np
import pytest
import torch

from helpers import TOL, batched_trace, run_trace, tail_trace, whole_trace
from plain_llama import PlainModel

pytestmark = pytest.mark.gpu


def _random_config(rng, wide=False):
    """``wide``: heads of 64 or 128 in groups of 10, 12 or 16 per kv head, which the tensor-core decode kernel takes
    as two blocks of instruction columns or as two warps per ring of pages."""
    from exl3_server_b200 import LlamaConfig
    hd = rng.choice([64, 128]) if wide else rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128])
    kvh = rng.choice([1, 2]) if wide else rng.choice([1, 2, 3, 4])
    heads = kvh * (rng.choice([10, 12, 16, 16]) if wide else rng.choice([1, 1, 2, 3, 4, 8]))
    hidden = rng.choice([64, 72, 96, 100, 136, 200, 256])
    layers = rng.choice([1, 2, 3])
    kw = dict(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kvh,
              head_dim=hd, intermediate_size=rng.choice([48, 100, 176, 208, 272, 333]),
              vocab_size=rng.choice([97, 256, 301, 1000, 2049]), tie_word_embeddings=rng.random() < 0.5,
              rope_theta=rng.choice([10000.0, 500000.0, 2500.0]), rms_norm_eps=rng.choice([1e-5, 1e-6, 3e-5]),
              max_position_embeddings=4096)
    if rng.random() < 0.5:
        kw.update(scale_emb=rng.choice([2.0, 12.0]), scale_depth=rng.choice([1.0, 1.4]),
                  dim_model_base=rng.choice([32, hidden // 2]))
    window = rng.choice([None, None, 20, 70, 150, 300] if wide else [None, None, 20, 70, 150])
    if window:
        kw.update(sliding_window=window,
                  layer_types=[rng.choice(["sliding_attention", "full_attention"]) for _ in range(layers)])
    return LlamaConfig(**kw), rng.random() < 0.3


@pytest.mark.parametrize("seed,wide", [(s, False) for s in (11, 12, 13, 14, 15, 16, 17, 18)] +
                         [(s, True) for s in (31, 32, 33, 34)])
def test_a_random_configuration(tmp_path, seed, wide):
    from exl3_server_b200 import Engine, write_random_model
    rng = random.Random(seed)
    cfg, biases = _random_config(rng, wide)
    folder = str(tmp_path / "model")
    write_random_model(cfg, folder, seed=seed, std=0.08, norm_std=0.1, dtype=torch.bfloat16, with_optional=biases)
    pm = PlainModel(folder)
    lens = [rng.choice([65, 200, 333, 400, 449, 520] if wide else [1, 2, 31, 64, 65, 129, 200, 333]) for _ in range(4)]
    reqs = {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n)] for i, n in enumerate(lens)}
    want = {k: pm.logits(v).numpy() for k, v in reqs.items()}
    ids = list(reqs)
    prompt_len = {r: max(1, len(reqs[r]) - k) for r, k in zip(ids, (3, 16, 0, 40))}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048)
        for what, trace in (("whole", whole_trace(reqs)), ("last 20 one by one", tail_trace(reqs, 20)),
                            ("batched", batched_trace(reqs, [[ids[0], ids[1], ids[2]], [ids[3], ids[0]]], prompt_len))):
            got = run_trace(eng, trace)
            for rid in got:
                assert np.isfinite(got[rid]).all(), (cfg, dtype, what, rid)
                err = float(np.max(np.abs(got[rid] - want[rid])) / np.max(np.abs(want[rid])))
                assert err <= TOL[dtype], f"{cfg}: {dtype} {what} {rid} (length {len(reqs[rid])}): {err:.3e}"
        assert eng.cache.tokens_held() == 0
