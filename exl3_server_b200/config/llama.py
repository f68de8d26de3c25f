"""Typed configuration of the Llama-family decoder (MiniCPM variant included).

Keys and defaults follow the reference's ``ModelConfig::load``
(src/model.cpp:97-118): ``hidden_size``, ``num_hidden_layers``,
``num_attention_heads``, ``intermediate_size`` and ``vocab_size`` are required;
``num_key_value_heads`` defaults to the head count, ``head_dim`` to
``hidden_size / heads``, ``rms_norm_eps`` to 1e-6, ``rope_theta`` to 10000,
``eos_token_id`` may be an integer or a list, and a non-null ``rope_scaling``
is refused.  The reference checks ``hidden_size % heads`` (src/model.cpp:180-183).

MiniCPM's constants have no counterpart in the reference's forward pass and are
read here: ``scale_emb`` multiplies the embedding, ``scale_depth / sqrt(layers)``
multiplies every sublayer output before the residual add, and the normed hidden
state is divided by ``hidden_size / dim_model_base`` before the head.  Absent
keys give factors of one, which is the reference's arithmetic.  Also read:
``tie_word_embeddings`` (absent: the head is tied exactly when the checkpoint has no ``lm_head.weight``),
``sliding_window`` with ``layer_types`` (a window of
keys for the layers marked ``"sliding_attention"``), ``hidden_act`` (must be
``"silu"``: the reference applies SiLU unconditionally, src/model.cpp:585).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .fields import ConfigError, KeyReader

LAYER_TYPES = ("full_attention", "sliding_attention")


@dataclass
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    vocab_size: int
    num_key_value_heads: int = 0          # 0: same as num_attention_heads
    head_dim: int = 0                     # 0: hidden_size // num_attention_heads
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 0
    bos_token_id: Optional[int] = None
    eos_token_id: List[int] = field(default_factory=list)
    scale_emb: float = 1.0
    scale_depth: Optional[float] = None   # None: sublayer outputs are not scaled
    dim_model_base: int = 0               # 0: hidden_size (divisor 1)
    tie_word_embeddings: Optional[bool] = None   # None: tied iff the checkpoint has no lm_head.weight
    sliding_window: Optional[int] = None
    layer_types: Optional[List[str]] = None
    model_type: str = "llama"
    architectures: List[str] = field(default_factory=lambda: ["LlamaForCausalLM"])

    def __post_init__(self) -> None:
        if self.num_key_value_heads == 0:
            self.num_key_value_heads = self.num_attention_heads
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "intermediate_size", "vocab_size"):
            if int(getattr(self, key)) < 1:
                raise ConfigError(f"config.json: key '{key}' must be >= 1, got {getattr(self, key)}")
        if self.head_dim == 0:
            if self.hidden_size % self.num_attention_heads != 0:
                raise ConfigError("config.json: hidden_size is not divisible by num_attention_heads")
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.dim_model_base == 0:
            self.dim_model_base = self.hidden_size
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "config.json: num_attention_heads (%d) is not a multiple of num_key_value_heads (%d)"
                % (self.num_attention_heads, self.num_key_value_heads))
        if self.head_dim % 16 != 0:
            # the rotation needs an even size; this engine's attention kernels take heads in steps of 16
            raise ConfigError(f"config.json: key 'head_dim' must be a multiple of 16, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: key 'rms_norm_eps' must be > 0")
        if not self.rope_theta > 0:
            raise ConfigError("config.json: key 'rope_theta' must be > 0")
        if self.sliding_window is not None and self.sliding_window < 1:
            raise ConfigError("config.json: key 'sliding_window' must be >= 1 or null")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError("config.json: layer_types does not match num_hidden_layers")
            for t in self.layer_types:
                if t not in LAYER_TYPES:
                    raise ConfigError(f"config.json: layer type {t!r} is not one of {LAYER_TYPES}")
            if "sliding_attention" in self.layer_types and self.sliding_window is None:
                raise ConfigError("config.json: layer_types names sliding_attention but sliding_window is null")

    # derived constants ------------------------------------------------------
    @property
    def residual_scale(self) -> float:
        if self.scale_depth is None:
            return 1.0
        return self.scale_depth / math.sqrt(self.num_hidden_layers)

    @property
    def logit_divisor(self) -> float:
        return self.hidden_size / self.dim_model_base

    def layer_window(self, i: int) -> int:
        """Keys that layer ``i`` may look back over; 0 means all of them."""
        if self.sliding_window is None:
            return 0
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[i] == "sliding_attention" else 0

    # JSON -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: Dict[str, Any]) -> "LlamaConfig":
        r = KeyReader(obj)
        if r.has("rope_scaling"):
            raise ConfigError("config.json: rope_scaling is not supported by this engine")
        act = r.string("hidden_act", None)
        if act is not None and act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        layer_types = r.raw("layer_types", None)
        if layer_types is not None and (
                not isinstance(layer_types, list) or not all(isinstance(t, str) for t in layer_types)):
            raise ConfigError("config.json: key 'layer_types' must be a list of strings")
        archs = r.raw("architectures", None)
        if archs is not None and (not isinstance(archs, list) or not all(isinstance(a, str) for a in archs)):
            raise ConfigError("config.json: key 'architectures' must be a list of strings")
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        return cls(
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            vocab_size=r.integer("vocab_size", minimum=1),
            num_key_value_heads=r.integer("num_key_value_heads", heads, minimum=1),
            head_dim=r.integer("head_dim", 0, minimum=0),
            rms_norm_eps=r.number("rms_norm_eps", 1e-6, positive=True),
            rope_theta=r.number("rope_theta", 10000.0, positive=True),
            max_position_embeddings=r.integer("max_position_embeddings", 0, minimum=0),
            bos_token_id=r.integer("bos_token_id", None),
            eos_token_id=r.int_list("eos_token_id", None),
            scale_emb=r.number("scale_emb", 1.0),
            scale_depth=r.number("scale_depth", None),
            dim_model_base=r.integer("dim_model_base", 0, minimum=0),
            tie_word_embeddings=r.boolean("tie_word_embeddings", None),
            sliding_window=r.integer("sliding_window", None),
            layer_types=layer_types,
            model_type=r.string("model_type", "llama"),
            architectures=list(archs) if archs else ["LlamaForCausalLM"],
        )

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu",
            "scale_emb": self.scale_emb,
            "dim_model_base": self.dim_model_base,
        }
        if self.tie_word_embeddings is not None:
            d["tie_word_embeddings"] = self.tie_word_embeddings
        if self.scale_depth is not None:
            d["scale_depth"] = self.scale_depth
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        return d
