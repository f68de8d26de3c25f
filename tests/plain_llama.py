"""A plain, slow implementation of the Llama-family decoder (MiniCPM constants
included): whole sequences, no cache, float64, one function per part.

It shares no code with the package: it reads config.json with ``json`` and the
weights with the ``safetensors`` library, and computes everything with plain
torch tensor arithmetic on the CPU.

It rests on the formulas, not on a run of the reference: the reference's model
code (src/model.cpp) needs Apple's MLX array library, which cannot be built or
imported on this machine, so there is no golden output of the reference's own
forward pass.  Each function cites the lines it restates.  The reference has no
``scale_emb`` / ``scale_depth`` / ``dim_model_base`` / tied head; with those at
their neutral values the arithmetic below is src/model.cpp:529-592 line by line.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch
from safetensors import safe_open

F = torch.float64


def read_config(model_dir: str) -> dict:
    """Keys and defaults of src/model.cpp:97-118, plus the MiniCPM constants."""
    with open(os.path.join(model_dir, "config.json")) as f:
        j = json.load(f)
    c = {
        "hidden": j["hidden_size"], "layers": j["num_hidden_layers"], "heads": j["num_attention_heads"],
        "inter": j["intermediate_size"], "vocab": j["vocab_size"],
    }
    c["kv_heads"] = j.get("num_key_value_heads", c["heads"])                    # model.cpp:100
    c["head_dim"] = j.get("head_dim") or c["hidden"] // c["heads"]              # model.cpp:101
    c["eps"] = j.get("rms_norm_eps", 1e-6)                                      # model.cpp:104
    c["theta"] = j.get("rope_theta", 10000.0)                                   # model.cpp:105
    c["scale_emb"] = j.get("scale_emb", 1.0)
    depth = j.get("scale_depth")
    c["rho"] = 1.0 if depth is None else depth / math.sqrt(c["layers"])
    c["divisor"] = c["hidden"] / (j.get("dim_model_base") or c["hidden"])
    c["tied"] = j.get("tie_word_embeddings")        # None: tied iff the checkpoint has no lm_head.weight
    window = j.get("sliding_window")
    types = j.get("layer_types")
    c["windows"] = [0 if window is None or (types is not None and types[i] != "sliding_attention") else window
                    for i in range(c["layers"])]
    return c


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(F)
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """h[t] = E[id_t] (src/model.cpp:529), times scale_emb."""
    return table[ids] * scale


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w (src/model.cpp:556, 582, 589: mx::fast::rms_norm)."""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x W^T + b with W stored (out, in) (src/model.cpp:549-552; bias iff present, :370-376)."""
    y = x @ w.T
    return y if b is None else y + b


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotation over the whole head (src/model.cpp:566-567: dims = head_dim,
    traditional = false, base = theta, scale = 1, offset = position).  x: [heads, L, hd]."""
    hd = x.shape[-1]
    half = hd // 2
    d = torch.arange(half, dtype=F)
    freq = theta ** (-2.0 * d / hd)
    a = positions.to(F)[:, None] * freq[None, :]                 # [L, half]
    cos, sin = torch.cos(a), torch.sin(a)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """softmax(q k^T / sqrt(hd) + causal mask) v with grouped heads
    (src/model.cpp:539-548 mask and scale, :576-578).  q: [heads, L, hd]; k, v: [kv_heads, L, hd]."""
    heads, L, hd = q.shape
    group = heads // k.shape[0]
    k = k.repeat_interleave(group, dim=0)                        # query head h reads kv head h // group
    v = v.repeat_interleave(group, dim=0)
    s = (q @ k.transpose(1, 2)) * (1.0 / math.sqrt(hd))
    i = torch.arange(L)[:, None]
    j = torch.arange(L)[None, :]
    allow = j <= i                                               # key position <= query position
    if window > 0:
        allow = allow & (j > i - window)
    s = s.masked_fill(~allow, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def swiglu(r: torch.Tensor, wg, wu, wd, bg=None, bu=None, bd=None) -> torch.Tensor:
    """(g * sigmoid(g) * u) Wd^T (src/model.cpp:583-586)."""
    g, u = linear(r, wg, bg), linear(r, wu, bu)
    return linear(g * torch.sigmoid(g) * u, wd, bd)


def layer(h: torch.Tensor, w: Dict[str, torch.Tensor], i: int, c: dict) -> torch.Tensor:
    """One pre-norm layer (src/model.cpp:554-587) with the residual scale rho."""
    p = f"model.layers.{i}."
    L = h.shape[0]
    pos = torch.arange(L)
    r = rms_norm(h, w[p + "input_layernorm.weight"], c["eps"])
    a = p + "self_attn."
    q = linear(r, w[a + "q_proj.weight"], w.get(a + "q_proj.bias"))
    k = linear(r, w[a + "k_proj.weight"], w.get(a + "k_proj.bias"))
    v = linear(r, w[a + "v_proj.weight"], w.get(a + "v_proj.bias"))
    q = q.view(L, c["heads"], c["head_dim"]).transpose(0, 1)     # model.cpp:562-564
    k = k.view(L, c["kv_heads"], c["head_dim"]).transpose(0, 1)
    v = v.view(L, c["kv_heads"], c["head_dim"]).transpose(0, 1)
    q, k = rope(q, pos, c["theta"]), rope(k, pos, c["theta"])
    o = attention(q, k, v, c["windows"][i]).transpose(0, 1).reshape(L, -1)      # model.cpp:579
    h = h + linear(o, w[a + "o_proj.weight"], w.get(a + "o_proj.bias")) * c["rho"]   # model.cpp:580
    r = rms_norm(h, w[p + "post_attention_layernorm.weight"], c["eps"])
    m = p + "mlp."
    y = swiglu(r, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"],
               w.get(m + "gate_proj.bias"), w.get(m + "up_proj.bias"), w.get(m + "down_proj.bias"))
    return h + y * c["rho"]                                      # model.cpp:586


def forward(w: Dict[str, torch.Tensor], c: dict, ids: List[int]) -> torch.Tensor:
    """Logits [L, vocab] of one whole sequence (src/model.cpp:514-592)."""
    t = torch.tensor(ids, dtype=torch.long)
    h = embedding(t, w["model.embed_tokens.weight"], c["scale_emb"])
    for i in range(c["layers"]):
        h = layer(h, w, i, c)
    h = rms_norm(h, w["model.norm.weight"], c["eps"]) / c["divisor"]
    tied = c["tied"] if c["tied"] is not None else "lm_head.weight" not in w
    head = w["model.embed_tokens.weight"] if tied else w["lm_head.weight"]
    return linear(h, head)


class PlainModel:
    def __init__(self, model_dir: str):
        self.c = read_config(model_dir)
        self.w = read_weights(model_dir)

    def logits(self, ids: List[int]) -> torch.Tensor:
        return forward(self.w, self.c, ids)

    def greedy(self, ids: List[int], n: int) -> List[int]:
        """n greedy tokens after the prompt; first maximum wins (src/model.cpp:688-696)."""
        ids = list(ids)
        out = []
        for _ in range(n):
            nxt = int(torch.argmax(self.logits(ids)[-1]))
            out.append(nxt)
            ids.append(nxt)
        return out
