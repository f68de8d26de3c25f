"""Configuration parsing, defaults, errors and the architecture registry."""
import json
import math

import pytest

from exl3_server_b200 import ConfigError, LlamaConfig
from exl3_server_b200.config import (read_config_json, register_architecture, registered_names,
                                     resolve_architecture, unregister_architecture)
from exl3_server_b200.models.llama import build_plan

REQUIRED = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=176, vocab_size=256)


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_dict(dict(REQUIRED))
    assert c.num_key_value_heads == 4            # defaults to the head count
    assert c.head_dim == 16                      # hidden / heads
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.scale_emb == 1.0 and c.residual_scale == 1.0 and c.logit_divisor == 1.0
    assert c.tie_word_embeddings is None and c.eos_token_id == [] and c.bos_token_id is None


@pytest.mark.parametrize("key", list(REQUIRED))
def test_missing_required_key_is_named(key):
    d = dict(REQUIRED)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(d)


def test_minicpm_constants():
    c = LlamaConfig.from_dict({**REQUIRED, "scale_emb": 12, "scale_depth": 1.4, "dim_model_base": 32,
                               "tie_word_embeddings": True})
    assert c.scale_emb == 12.0
    assert c.residual_scale == pytest.approx(1.4 / math.sqrt(2))
    assert c.logit_divisor == 2.0
    plan = build_plan(c)
    assert plan.head.tied and plan.head.input_divisor == 2.0 and plan.embedding.scale == 12.0
    assert all(layer.residual_scale == c.residual_scale for layer in plan.layers)


def test_eos_as_integer_or_list():
    assert LlamaConfig.from_dict({**REQUIRED, "eos_token_id": 7}).eos_token_id == [7]
    assert LlamaConfig.from_dict({**REQUIRED, "eos_token_id": [7, 9]}).eos_token_id == [7, 9]


@pytest.mark.parametrize("patch, word", [
    ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"hidden_size": 66, "head_dim": 0}, "divisible"),
    ({"head_dim": 15}, "'head_dim' must be a multiple of 16"),
    ({"head_dim": 24}, "'head_dim' must be a multiple of 16"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding_window"),
    ({"layer_types": ["full_attention", "strided"], "sliding_window": 8}, "strided"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_errors_name_the_key(patch, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict({**REQUIRED, **patch})


def test_window_per_layer():
    c = LlamaConfig.from_dict({**REQUIRED, "sliding_window": 8,
                               "layer_types": ["sliding_attention", "full_attention"]})
    plan = build_plan(c)
    assert [layer.mixer.window for layer in plan.layers] == [8, 0]
    c = LlamaConfig.from_dict({**REQUIRED, "sliding_window": 8})
    assert [layer.mixer.window for layer in build_plan(c).layers] == [8, 8]


def test_round_trip_through_json(tmp_path):
    c = LlamaConfig.from_dict({**REQUIRED, "scale_depth": 1.4, "eos_token_id": [1, 2], "sliding_window": 16})
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    again = LlamaConfig.from_dict(read_config_json(str(tmp_path)))
    assert again == c


def test_bad_json_and_missing_file(tmp_path):
    with pytest.raises(ConfigError, match="no such file"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_registry_names_and_unknown():
    for name in ("LlamaForCausalLM", "llama", "MiniCPMForCausalLM", "minicpm"):
        assert name in registered_names()
    a = resolve_architecture({"architectures": ["MiniCPMForCausalLM"], "model_type": "whatever"})
    assert a.config_class is LlamaConfig
    assert resolve_architecture({"model_type": "llama"}).build_plan is build_plan
    with pytest.raises(ConfigError, match="registered: .*llama"):
        resolve_architecture({"architectures": ["GptOssForCausalLM"], "model_type": "gpt_oss"})
    with pytest.raises(ConfigError, match="neither"):
        resolve_architecture({})


def test_registering_another_architecture():
    class Cfg:
        @classmethod
        def from_dict(cls, d):
            return cls()

    try:
        register_architecture(["ToyForCausalLM", "toy"], Cfg, lambda cfg: "plan")
        assert resolve_architecture({"model_type": "toy"}).build_plan(None) == "plan"
    finally:
        unregister_architecture(["ToyForCausalLM", "toy"])
    with pytest.raises(ConfigError):
        resolve_architecture({"model_type": "toy"})


def test_plan_schedule_validation():
    from exl3_server_b200.parts import ScheduleEntry
    plan = build_plan(LlamaConfig.from_dict(dict(REQUIRED)))
    plan.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_from=0)]
    plan.validate()                                  # a layer twice, reading an earlier cache: fine
    plan.schedule = [ScheduleEntry(0), ScheduleEntry(5)]
    with pytest.raises(ValueError, match="names layer 5"):
        plan.validate()
    plan.schedule = [ScheduleEntry(0, cache_from=0)]
    with pytest.raises(ValueError, match="earlier entry"):
        plan.validate()
