"""The engine against the plain implementation at layer sizes of real models (two layers of each, random
weights): the benchmark's MiniCPM-2B sizes (36 heads of 64, width 2304, vocabulary 122753, tied head),
Llama-3-8B-like sizes (32 query heads on 8 key/value heads of 128, width 4096, feed-forward 14336, vocabulary
128256) and the MiniCPM4-8B sizes (32 query heads on 2 key/value heads of 128: 16 query heads share a key/value
head; feed-forward 16384).  The tiny configurations of the other tests reach every option; these reach the shapes
the kernels are tuned for: whole prompt, then the last 40 tokens one by one, then a batch of 24 decoding
together (more than the 16 rows the weight-streaming projection takes)."""
import numpy as np
import pytest
import torch

from helpers import TOL, run_trace, tail_trace, whole_trace
from plain_llama import PlainModel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["minicpm-2b", "llama-8b-like", "minicpm4-8b"])
def test_two_layers_of_real_sizes(tmp_path, name):
    from exl3_server_b200 import Engine, LlamaConfig, write_random_model
    from exl3_server_b200.config.presets import sizes
    cfg = LlamaConfig(**sizes(name, num_hidden_layers=2))
    folder = str(tmp_path / name)
    write_random_model(cfg, folder, seed=3, std=0.02)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg.vocab_size, (200,), generator=g).tolist()
    want = PlainModel(folder).logits(toks).numpy()
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=8192)
        for what, trace in (("whole", whole_trace({"r0": toks})), ("last 40 one by one", tail_trace({"r0": toks}, tail=40))):
            got = run_trace(eng, trace)["r0"]
            per_pos = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
            bad = np.nonzero(per_pos > TOL[dtype])[0]
            assert bad.size == 0, f"{name} {dtype} {what}: first wrong position {bad[0]}, error {per_pos[bad[0]]:.3e}"
        if dtype == "bfloat16":
            # 24 copies of the request's first 160 tokens, then 40 steps of all 24 rows: every row must follow
            # the plain implementation's logits for the request
            from exl3_server_b200 import StepEntry
            slots = [eng.open() for _ in range(24)]
            eng.step([StepEntry(s, toks[:160], None) for s in slots])
            session = eng.decode_session(slots, max_new=64)
            for p in range(160, 200):
                got = session.step([toks[p]] * 24).float().cpu().numpy()
                err = np.max(np.abs(got - want[p][None]), axis=1).max() / np.max(np.abs(want[p]))
                assert err <= TOL[dtype], f"{name}: 24 rows at position {p}: error {err:.3e}"
            session.close()
            for s in slots:
                eng.close(s)
        del eng
        torch.cuda.empty_cache()


def test_long_prompts_through_the_paired_projections(tmp_path, monkeypatch):
    """Two prompts of 2,047 and 1,501 tokens in one step at the MiniCPM-2B layer sizes (a small vocabulary, so that
    the plain implementation is done in seconds): rows enough for the paired tcgen05 GEMM with the norms, the
    residual, the rotary encoding and the cache write in its epilogues; the second prompt starts in the middle of
    a tile and of a warp's rows, so its keys and values go to the cache by the epilogue's other path.  Then both
    go on token by token from that cache."""
    from exl3_server_b200 import Engine, LlamaConfig, write_random_model
    from exl3_server_b200.config.presets import sizes
    from exl3_server_b200.ops import kernels as K
    from helpers import batched_trace
    cfg = LlamaConfig(**sizes("minicpm-2b", num_hidden_layers=2, vocab_size=1000))
    folder = str(tmp_path / "m")
    write_random_model(cfg, folder, seed=4, std=0.02)
    g = torch.Generator().manual_seed(3)
    reqs = {"a": torch.randint(0, cfg.vocab_size, (2047 + 6,), generator=g).tolist(),
            "b": torch.randint(0, cfg.vocab_size, (1501 + 6,), generator=g).tolist()}
    plain = PlainModel(folder)
    want = {rid: plain.logits(t).numpy() for rid, t in reqs.items()}
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=8192)
    calls = {"rotated": 0, "into the residual": 0, "gated": 0}
    rope, pair = K.gemm_pair_rope, K.gemm_pair

    def counted_rope(*a, **k):
        calls["rotated"] += 1
        return rope(*a, **k)

    def counted_pair(*a, **k):
        calls["into the residual"] += k.get("resid") is not None
        calls["gated"] += bool(k.get("gated"))
        return pair(*a, **k)

    monkeypatch.setattr(K, "gemm_pair_rope", counted_rope)
    monkeypatch.setattr(K, "gemm_pair", counted_pair)
    got = run_trace(eng, batched_trace(reqs, [["a", "b"]], {"a": 2047, "b": 1501}))
    # per layer: q/k/v with the position step, o and down into the residual (the last down has no norm after it
    # inside the block), gate/up with the activation
    assert calls == {"rotated": 2, "into the residual": 3, "gated": 2}, calls
    for rid in reqs:
        per_pos = np.max(np.abs(got[rid] - want[rid]), axis=1) / np.max(np.abs(want[rid]))
        bad = np.nonzero(per_pos > TOL["bfloat16"])[0]
        assert bad.size == 0, f"request {rid}: first wrong position {bad[0]}, error {per_pos[bad[0]]:.3e}"
    K.check_status()


@pytest.mark.parametrize("name,tokens,form", [("minicpm-2b", 2048, 3), ("minicpm-2b", 1536, 1), ("minicpm4-8b", 1100, None)])
def test_a_long_prompt_in_each_form_of_the_prompt_attention(tmp_path, monkeypatch, name, tokens, form):
    """One prompt whose tiles the tensor-core attention walks two a block (2,048 tokens at the MiniCPM-2B sizes: 576
    blocks would be two rounds) or one a block (1,536 tokens: the heaviest tile is the kernel's length anyway), and
    one with heads of 128: every logit against the plain implementation, and the form that the attention part
    asked for."""
    from exl3_server_b200 import Engine, LlamaConfig, write_random_model
    from exl3_server_b200.config.presets import sizes
    from exl3_server_b200.ops import kernels as K
    cfg = LlamaConfig(**sizes(name, num_hidden_layers=2, vocab_size=1000))
    folder = str(tmp_path / "m")
    write_random_model(cfg, folder, seed=6, std=0.02)
    g = torch.Generator().manual_seed(8)
    toks = torch.randint(0, cfg.vocab_size, (tokens,), generator=g).tolist()
    want = PlainModel(folder).logits(toks).numpy()
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=4096)
    asked = []
    kernel = K.attn_prefill_tc

    def watched(*a, **k):
        asked.append(k.get("variant", 0))
        return kernel(*a, **k)

    monkeypatch.setattr(K, "attn_prefill_tc", watched)
    got = run_trace(eng, whole_trace({"r0": toks}))["r0"]
    assert len(asked) == 2 and (form is None or asked == [form, form]), asked
    assert K.attn_prefill_tc_status() == 0
    per_pos = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
    bad = np.nonzero(per_pos > TOL["bfloat16"])[0]
    assert bad.size == 0, f"first wrong position {bad[0]}, error {per_pos[bad[0]]:.3e}"
