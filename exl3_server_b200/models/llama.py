"""The Llama-family decoder (MiniCPM constants included) as a plan of parts.

Tensor names are the checkpoint's own, as the reference reads them
(src/model.cpp:379-416): ``model.embed_tokens.weight``, ``model.norm.weight``,
``lm_head.weight`` and, per layer ``model.layers.{i}``, ``input_layernorm``,
``self_attn.{q,k,v,o}_proj``, ``post_attention_layernorm``,
``mlp.{gate,up,down}_proj``.  Every layer is pre-norm attention + SwiGLU
(src/model.cpp:554-587); the layers run once each, in order.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan, NormSpec,
                          PositionSpec, ScheduleEntry)

NAMES = ("LlamaForCausalLM", "llama", "MiniCPMForCausalLM", "minicpm", "MiniCPM5ForCausalLM", "minicpm5",
         "MistralForCausalLM", "mistral")


def build_plan(cfg: LlamaConfig) -> ModelPlan:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            arrangement="prenorm",
            mixer=MixerSpec(
                kind="attention", width=cfg.hidden_size, heads=cfg.num_attention_heads,
                kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, window=cfg.layer_window(i),
                position=PositionSpec(kind="rope", dims=cfg.head_dim, theta=cfg.rope_theta, scale=1.0)),
            feed_forward=FeedForwardSpec(kind="swiglu", width=cfg.hidden_size, inner=cfg.intermediate_size),
            mixer_norm=NormSpec(kind="rms", width=cfg.hidden_size, eps=cfg.rms_norm_eps),
            feed_forward_norm=NormSpec(kind="rms", width=cfg.hidden_size, eps=cfg.rms_norm_eps),
            residual_scale=cfg.residual_scale,
            names={"mixer": p + "self_attn.", "feed_forward": p + "mlp.",
                   "mixer_norm": p + "input_layernorm.", "feed_forward_norm": p + "post_attention_layernorm."},
        ))
    plan = ModelPlan(
        architecture=cfg.architectures[0] if cfg.architectures else cfg.model_type,
        embedding=EmbeddingSpec(vocab=cfg.vocab_size, width=cfg.hidden_size, scale=cfg.scale_emb,
                                name="model.embed_tokens.weight"),
        layers=layers,
        schedule=[ScheduleEntry(layer=i) for i in range(cfg.num_hidden_layers)],
        final_norm=NormSpec(kind="rms", width=cfg.hidden_size, eps=cfg.rms_norm_eps),
        final_norm_name="model.norm.",
        head=HeadSpec(vocab=cfg.vocab_size, width=cfg.hidden_size, input_divisor=cfg.logit_divisor,
                      tied=cfg.tie_word_embeddings, name="lm_head.weight"),
        max_positions=cfg.max_position_embeddings,
        stop_token_ids=list(cfg.eos_token_id),
        bos_token_id=cfg.bos_token_id,
        ignorable=["*.rotary_emb.inv_freq"],      # stored by older exporters; the angles are computed here
    )
    plan.validate()
    return plan


register_architecture(NAMES, LlamaConfig, build_plan)
