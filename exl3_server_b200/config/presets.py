"""Layer sizes of real models, for benchmarks and for tests at the shapes the kernels are tuned for.  No model
code looks here: a model's sizes come from its own config.json; these tables only save a benchmark or a test
from repeating them.  Each entry is the keyword arguments of ``LlamaConfig``.

``minicpm-2b``: MiniCPM-2B; ``minicpm4-0.5b`` and ``minicpm4-8b``: the MiniCPM4 sizes (grouped heads, 16 query
heads per key/value head in the larger one); ``llama-8b-like``: Llama-3-8B's layer sizes.
"""
from __future__ import annotations

from typing import Any, Dict

_MINICPM = dict(rope_theta=10000.0, scale_emb=12.0, scale_depth=1.4, dim_model_base=256,
                max_position_embeddings=0, model_type="minicpm", architectures=["MiniCPMForCausalLM"])

SIZES: Dict[str, Dict[str, Any]] = {
    "minicpm-2b": dict(hidden_size=2304, num_hidden_layers=40, num_attention_heads=36, num_key_value_heads=36,
                       head_dim=64, intermediate_size=5760, vocab_size=122753, tie_word_embeddings=True,
                       rms_norm_eps=1e-5, **_MINICPM),
    "minicpm4-0.5b": dict(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, num_key_value_heads=2,
                          head_dim=64, intermediate_size=4096, vocab_size=73448, tie_word_embeddings=True,
                          rms_norm_eps=1e-5, **_MINICPM),
    "minicpm4-8b": dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=2,
                        head_dim=128, intermediate_size=16384, vocab_size=73448, tie_word_embeddings=False,
                        rms_norm_eps=1e-6, **_MINICPM),
    "llama-8b-like": dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                          head_dim=128, intermediate_size=14336, vocab_size=128256, tie_word_embeddings=False,
                          rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=0),
}


def sizes(name: str, **overrides: Any) -> Dict[str, Any]:
    """The named table with some keys replaced (``num_hidden_layers=2`` for a test)."""
    try:
        base = SIZES[name]
    except KeyError:
        raise KeyError(f"no size table named {name!r}; known: {sorted(SIZES)}") from None
    return {**base, **overrides}
