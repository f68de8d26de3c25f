"""The safetensors container, binding by name and its one error, random weights."""
import json
import os
import struct

import pytest
import torch

from exl3_server_b200 import LlamaConfig, WeightsError, write_random_model
from exl3_server_b200.engine.model import plan_manifest
from exl3_server_b200.models.llama import build_plan
from exl3_server_b200.weights import (TensorSpec, TensorStore, check_manifest, load_tensors, stored_dtype,
                                      write_safetensors)

CFG = LlamaConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=48, vocab_size=50,
                  tie_word_embeddings=False)


def test_round_trip_and_foreign_reader(tmp_path):
    path = str(tmp_path / "model.safetensors")
    tensors = [("a", torch.randn(3, 5).to(torch.bfloat16)), ("b", torch.arange(7, dtype=torch.int32)),
               ("c", torch.randn(4).to(torch.float32)), ("d", torch.randn(2, 2).to(torch.float16))]
    write_safetensors(path, tensors)
    store = TensorStore(str(tmp_path))
    for name, t in tensors:
        assert torch.equal(store.tensor(name), t)
    from safetensors import safe_open                    # an independent reader agrees
    with safe_open(path, framework="pt") as f:
        assert sorted(f.keys()) == ["a", "b", "c", "d"]
        for name, t in tensors:
            assert torch.equal(f.get_tensor(name), t)


def test_reads_what_the_safetensors_library_writes(tmp_path):
    from safetensors.torch import save_file
    t = {"x": torch.randn(4, 6).to(torch.bfloat16), "y": torch.ones(3)}
    save_file(t, str(tmp_path / "model.safetensors"))
    store = TensorStore(str(tmp_path))
    assert torch.equal(store.tensor("x"), t["x"]) and torch.equal(store.tensor("y"), t["y"])


def test_shards_through_the_index(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), [("a", torch.ones(2))])
    write_safetensors(str(tmp_path / "s2.safetensors"), [("b", torch.zeros(3))])
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    store = TensorStore(str(tmp_path))
    assert sorted(store.names()) == ["a", "b"] and store.shape("b") == (3,)


@pytest.mark.parametrize("damage, word", [
    (lambda raw: raw[:4], "truncated"),
    (lambda raw: struct.pack("<Q", 10 ** 9) + raw[8:], "header length"),
    (lambda raw: raw[:8] + b"{" * (len(raw) - 8), "bad safetensors header"),
    (lambda raw: raw[:-3], "inconsistent size"),
])
def test_corrupt_files(tmp_path, damage, word):
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, [("a", torch.ones(8))])
    raw = open(path, "rb").read()
    open(path, "wb").write(damage(raw))
    with pytest.raises(WeightsError, match=word):
        TensorStore(str(tmp_path))


def test_no_weights_in_folder(tmp_path):
    with pytest.raises(WeightsError, match="no model.safetensors"):
        TensorStore(str(tmp_path))


def test_storage_rule():
    bf, f32 = torch.bfloat16, torch.float32
    assert stored_dtype(torch.float16, "float", bf) == bf
    assert stored_dtype(torch.bfloat16, "float", bf) == bf
    assert stored_dtype(f32, "float", bf) == f32              # stored in 32-bit: stays so
    assert stored_dtype(torch.bfloat16, "float", f32) == f32  # the 32-bit path widens
    assert stored_dtype(torch.int64, "int", bf) == torch.int32
    with pytest.raises(WeightsError):
        stored_dtype(torch.int32, "float", bf)


def test_one_error_lists_everything(tmp_path):
    folder = write_random_model(CFG, str(tmp_path / "m"), seed=1)
    manifest = plan_manifest(build_plan(CFG))
    store = TensorStore(folder)
    tensors = {n: store.tensor(n).clone() for n in store.names()}
    del tensors["model.norm.weight"], tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(32, 31, dtype=torch.bfloat16)
    tensors["model.layers.0.rotary.inv_freq"] = torch.zeros(4)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, manifest, torch.bfloat16)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.norm.weight" in msg and "up_proj" in msg
    assert "unexpected tensors (1)" in msg and "rotary.inv_freq" in msg
    assert "wrong shapes (1)" in msg and "[32, 31], expected [32, 32]" in msg


def test_tied_head_needs_no_lm_head_and_refuses_a_stray_one(tmp_path):
    tied = LlamaConfig.from_dict({**CFG.to_dict(), "tie_word_embeddings": True})
    folder = write_random_model(tied, str(tmp_path / "t"), seed=1)
    names = TensorStore(folder).names()
    assert "lm_head.weight" not in names
    load_tensors(folder, plan_manifest(build_plan(tied)), torch.bfloat16)
    with pytest.raises(WeightsError, match="missing tensors.*lm_head.weight"):
        load_tensors(folder, plan_manifest(build_plan(CFG)), torch.bfloat16)
    untied = write_random_model(CFG, str(tmp_path / "u"), seed=1)
    with pytest.raises(WeightsError, match="unexpected tensors.*lm_head.weight"):
        load_tensors(untied, plan_manifest(build_plan(tied)), torch.bfloat16)


def test_an_absent_tie_key_follows_the_checkpoint(tmp_path):
    """config.json without ``tie_word_embeddings``: the head is the embedding table exactly when the checkpoint
    has no ``lm_head.weight``."""
    d = CFG.to_dict()
    del d["tie_word_embeddings"]
    free = LlamaConfig.from_dict(d)
    assert free.tie_word_embeddings is None and "tie_word_embeddings" not in free.to_dict()
    plan = build_plan(free)
    without = write_random_model(free, str(tmp_path / "w"), seed=1)          # optional tensors are not written
    assert "lm_head.weight" not in TensorStore(without).names()
    assert "lm_head.weight" not in load_tensors(without, plan_manifest(plan), torch.bfloat16)
    with_head = write_random_model(CFG, str(tmp_path / "h"), seed=1)
    assert "lm_head.weight" in load_tensors(with_head, plan_manifest(plan), torch.bfloat16)
    from exl3_server_b200.engine.engine import load_model
    assert load_model(without, "float32", "cpu").head.tied and not load_model(with_head, "float32", "cpu").head.tied


def test_tensors_the_architecture_declares_ignorable_may_be_there(tmp_path):
    folder = write_random_model(CFG, str(tmp_path / "m"), seed=1)
    plan = build_plan(CFG)
    store = TensorStore(folder)
    tensors = {n: store.tensor(n).clone() for n in store.names()}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    got = load_tensors(folder, plan_manifest(plan), torch.bfloat16, ignorable=plan.ignorable)
    assert not any("inv_freq" in n for n in got)
    with pytest.raises(WeightsError, match=r"unexpected tensors \(2\)"):
        load_tensors(folder, plan_manifest(plan), torch.bfloat16)            # without the plan's patterns
    tensors["model.layers.0.self_attn.extra.weight"] = torch.zeros(2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    with pytest.raises(WeightsError, match=r"unexpected tensors \(1\): model.layers.0.self_attn.extra.weight"):
        load_tensors(folder, plan_manifest(plan), torch.bfloat16, ignorable=plan.ignorable)


def test_optional_biases():
    manifest = [TensorSpec("w", (2, 2)), TensorSpec("b", (2,), optional=True)]
    check_manifest(manifest, {"w": (2, 2)})
    check_manifest(manifest, {"w": (2, 2), "b": (2,)})
    with pytest.raises(WeightsError, match="wrong shapes"):
        check_manifest(manifest, {"w": (2, 2), "b": (3,)})


def test_random_weights_are_seeded_per_tensor(tmp_path):
    a = TensorStore(write_random_model(CFG, str(tmp_path / "a"), seed=5))
    b = TensorStore(write_random_model(CFG, str(tmp_path / "b"), seed=5))
    c = TensorStore(write_random_model(CFG, str(tmp_path / "c"), seed=6))
    name = "model.layers.1.mlp.down_proj.weight"
    assert torch.equal(a.tensor(name), b.tensor(name))
    assert not torch.equal(a.tensor(name), c.tensor(name))
    w = a.tensor(name).float()
    assert abs(float(w.std()) - 0.02) < 0.004
    n = a.tensor("model.norm.weight").float()
    assert abs(float(n.mean()) - 1.0) < 0.02
    assert json.load(open(os.path.join(str(tmp_path / "a"), "config.json")))["hidden_size"] == 32


def test_float32_storage_is_kept(tmp_path):
    folder = write_random_model(CFG, str(tmp_path / "f"), seed=2, dtype=torch.float32)
    t = load_tensors(folder, plan_manifest(build_plan(CFG)), torch.bfloat16)
    assert all(v.dtype == torch.float32 for v in t.values())
