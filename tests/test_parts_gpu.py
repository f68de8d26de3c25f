"""Each part alone against the plain implementation's function for it, and a
toy architecture, defined here, that is registered, built and stepped without
any change to the framework: a mixer with per-sequence state of its own beside
attention layers, a layer that runs twice and a layer that reads another
layer's keys and values."""
import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import batched_trace, rel_err, run_trace, tail_trace, whole_trace

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def ctx(dtype):
    from exl3_server_b200.parts import BuildContext
    return BuildContext(dtype=dtype, device=DEV)


def one_sequence_batch(cache, n, start=0):
    """A step of n tokens for one fresh sequence (positions start..)."""
    from exl3_server_b200.engine.batch import Workspace, pack_step
    slot = cache.open()
    if start:
        cache.reserve({slot: start})
        cache.commit(slot, start)
    cache.reserve({slot: start + n})
    return pack_step([slot], [start], [[0] * n], [[n - 1]], cache.block_tables([slot]), Workspace(DEV), DEV), slot


TOLS = {torch.float32: 3e-6, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from exl3_server_b200.parts import NormSpec, ResidualStream, norm_class
    torch.manual_seed(0)
    H = 200
    w = (1 + 0.2 * torch.randn(H)).to(dtype)
    part = norm_class("rms")(NormSpec("rms", H, 3e-6), {"n.weight": w.to(DEV)}, "n.", ctx(dtype))
    h = torch.randn(5, H, device=DEV)
    y = torch.randn(5, H, device=DEV).to(dtype)
    stream = ResidualStream(h.clone())
    stream.push(y, 0.5)
    r = part.add_norm(stream)
    hn = h.double().cpu() + 0.5 * y.double().cpu()
    assert stream.pending is None and rel_err(stream.h.cpu().numpy(), hn.numpy()) < 1e-6
    assert rel_err(r.float().cpu().numpy(), P.rms_norm(hn, w.double(), 3e-6).numpy()) <= TOLS[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_position_part_and_cache_write(dtype):
    from exl3_server_b200.cache import SequenceCache
    from exl3_server_b200.parts import KVRequest, PositionSpec, position_class
    torch.manual_seed(1)
    nh, nkv, hd, n, start = 4, 2, 32, 70, 60
    cache = SequenceCache([(KVRequest(nkv, hd), None, None)], 512, dtype=dtype, device=DEV)
    batch, slot = one_sequence_batch(cache, n, start)
    part = position_class("rope")(PositionSpec("rope", dims=hd, theta=5000.0), hd, ctx(dtype))
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, device=DEV).to(dtype)
    orig = qkv.double().cpu()
    kv = cache.view(0, batch.block_tables)
    part.rotate_and_store(qkv, batch, kv, nh, nkv, hd)
    pos = torch.arange(start, start + n)
    q = orig[:, :nh * hd].view(n, nh, hd).transpose(0, 1)
    k = orig[:, nh * hd:(nh + nkv) * hd].view(n, nkv, hd).transpose(0, 1)
    v = orig[:, (nh + nkv) * hd:].view(n, nkv, hd)
    want_q = P.rope(q, pos, 5000.0).transpose(0, 1).reshape(n, -1)
    want_k = P.rope(k, pos, 5000.0)                     # [nkv, n, hd]
    # Angles are float32 by design: the frequency and the product pos * f are each rounded to
    # 24 bits, so an angle near position p is off by up to 2 * p * 2^-24 radians, and a rotated
    # value by that times its size.  The plain implementation's angles are float64.
    tol = max(TOLS[dtype], 2 * (start + n) * 2.0 ** -24)
    assert rel_err(qkv[:, :nh * hd].float().cpu().numpy(), want_q.numpy()) <= tol
    pages = cache.groups[0].pages[slot]
    for i, p in enumerate(range(start, start + n)):
        got_k = kv.k[pages[p // 64], :, p % 64].float().cpu()
        got_v = kv.v[pages[p // 64], :, p % 64].double().cpu()
        assert rel_err(got_k.numpy(), want_k[:, i].numpy()) <= tol
        assert torch.equal(got_v, v[i])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 20])
def test_attention_part(dtype, window):
    from exl3_server_b200.cache import SequenceCache
    from exl3_server_b200.parts import MixerSpec, PositionSpec, mixer_class
    torch.manual_seed(2)
    H, nh, nkv, hd, n = 72, 6, 2, 16, 90
    spec = MixerSpec("attention", width=H, heads=nh, kv_heads=nkv, head_dim=hd, window=window,
                     position=PositionSpec("rope", dims=hd, theta=300.0))
    names = {"q_proj": (nh * hd, H), "k_proj": (nkv * hd, H), "v_proj": (nkv * hd, H), "o_proj": (H, nh * hd)}
    t = {}
    for nm, shape in names.items():
        t[f"a.{nm}.weight"] = (torch.randn(shape) / math.sqrt(shape[1])).to(dtype).to(DEV)
        t[f"a.{nm}.bias"] = (0.1 * torch.randn(shape[0])).to(dtype).to(DEV)
    part = mixer_class("attention")(spec, t, "a.", ctx(dtype))
    cache = SequenceCache([(part.cache_request(), part.state_request(), None)], 512, dtype=dtype, device=DEV)
    batch, _ = one_sequence_batch(cache, n)
    x = torch.randn(n, H, device=DEV).to(dtype)
    y = part.forward(x, batch, cache.view(0, batch.block_tables), None)
    w = {k: v.double().cpu() for k, v in t.items()}
    xd = x.double().cpu()
    q = P.linear(xd, w["a.q_proj.weight"], w["a.q_proj.bias"]).view(n, nh, hd).transpose(0, 1)
    k = P.linear(xd, w["a.k_proj.weight"], w["a.k_proj.bias"]).view(n, nkv, hd).transpose(0, 1)
    v = P.linear(xd, w["a.v_proj.weight"], w["a.v_proj.bias"]).view(n, nkv, hd).transpose(0, 1)
    pos = torch.arange(n)
    o = P.attention(P.rope(q, pos, 300.0), P.rope(k, pos, 300.0), v, window).transpose(0, 1).reshape(n, -1)
    want = P.linear(o, w["a.o_proj.weight"], w["a.o_proj.bias"])
    assert rel_err(y.float().cpu().numpy(), want.numpy()) <= TOLS[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,rows", [(176, 3), (100, 3), (176, 40)])
def test_feed_forward_part(dtype, inner, rows):
    """inner 100 is not a multiple of 8 (plain layout); 40 rows take the large-batch path."""
    from exl3_server_b200.parts import FeedForwardSpec, feed_forward_class
    torch.manual_seed(3)
    H = 64
    t = {"f.gate_proj.weight": (torch.randn(inner, H) / 8).to(dtype).to(DEV),
         "f.up_proj.weight": (torch.randn(inner, H) / 8).to(dtype).to(DEV),
         "f.down_proj.weight": (torch.randn(H, inner) / 10).to(dtype).to(DEV),
         "f.gate_proj.bias": (0.1 * torch.randn(inner)).to(dtype).to(DEV)}
    part = feed_forward_class("swiglu")(FeedForwardSpec("swiglu", H, inner), t, "f.", ctx(dtype))
    x = torch.randn(rows, H, device=DEV).to(dtype)
    y = part.forward(x, None)
    w = {k: v.double().cpu() for k, v in t.items()}
    want = P.swiglu(x.double().cpu(), w["f.gate_proj.weight"], w["f.up_proj.weight"], w["f.down_proj.weight"],
                    bg=w["f.gate_proj.bias"])
    assert rel_err(y.float().cpu().numpy(), want.numpy()) <= TOLS[dtype]


@pytest.mark.parametrize("rows", [40, 300])
def test_feed_forward_between_two_norms_that_are_no_kernels(rows, monkeypatch):
    """The feed-forward takes the norm before it in two pieces and leaves the norm after it in two pieces, with its
    output already in the residual: for a decode batch (40 rows: the skinny GEMM) and for a prompt (300 rows: the
    paired GEMM, which a batch this small gets only because the test lowers its threshold)."""
    from exl3_server_b200.parts import FeedForwardSpec, NormSpec, ResidualStream, feed_forward_class, norm_class
    from exl3_server_b200.parts import linear as LIN
    from exl3_server_b200.parts.base import NormAfter, RawNormed
    monkeypatch.setattr(LIN, "PAIR_MIN_EFFICIENCY", 0.0)
    torch.manual_seed(5)
    dtype, H, inner, eps, rho = torch.bfloat16, 264, 176, 2e-6, 0.4
    t = {"f.gate_proj.weight": (torch.randn(inner, H) / 16).to(dtype).to(DEV),
         "f.up_proj.weight": (torch.randn(inner, H) / 16).to(dtype).to(DEV),
         "f.down_proj.weight": (torch.randn(H, inner) / 13).to(dtype).to(DEV)}
    part = feed_forward_class("swiglu")(FeedForwardSpec("swiglu", H, inner), t, "f.", ctx(dtype))
    w1 = (1 + 0.2 * torch.randn(H)).to(dtype)
    w2 = (1 + 0.2 * torch.randn(H)).to(dtype)
    after = norm_class("rms")(NormSpec("rms", H, eps), {"n.weight": w2.to(DEV)}, "n.", ctx(dtype))
    h0 = torch.randn(rows, H) * 2
    # the norm before, as a projection would have left it: h times the weight, and sums of squares in three pieces
    x_raw = (h0 * w1.float()).to(dtype).to(DEV)
    sq = (h0.double() ** 2)
    ss = torch.stack([sq[:, :100].sum(1), sq[:, 100:200].sum(1), sq[:, 200:].sum(1)], dim=1).float().to(DEV)
    stream = ResidualStream(h0.clone().to(DEV))
    then = NormAfter(stream, rho, after)
    y = part.forward(RawNormed(x_raw, ss, eps, H), None, then=then)
    assert y is None and then.done and stream.pending is None
    w = {k: v.double().cpu() for k, v in t.items()}
    r1 = P.rms_norm(h0.double(), w1.double(), eps)
    want_h = h0.double() + rho * P.swiglu(r1, w["f.gate_proj.weight"], w["f.up_proj.weight"], w["f.down_proj.weight"])
    assert rel_err(stream.h.cpu().numpy(), want_h.numpy()) < 3e-3
    left = after.add_norm(stream, raw_ok=True)
    assert isinstance(left, RawNormed)
    want_r = P.rms_norm(want_h, w2.double(), eps)
    assert rel_err(left.materialize().float().cpu().numpy(), want_r.numpy()) <= TOLS[dtype]
    # one row of it, as the last norm of a prompt asks for
    rows_wanted = torch.tensor([rows - 1], dtype=torch.int32, device=DEV)
    stream.normed = (after, left)
    one = after.add_norm(stream, rows=rows_wanted)
    assert rel_err(one.float().cpu().numpy(), want_r[rows - 1:].numpy()) <= TOLS[dtype]
    from exl3_server_b200.ops import kernels as K
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head(dtype):
    from exl3_server_b200.parts import EmbeddingSpec, HeadSpec, NormSpec, norm_class
    from exl3_server_b200.parts.embedding import Embedding, Head
    torch.manual_seed(4)
    V, H = 263, 96
    E = torch.randn(V, H).to(dtype)
    wn = (1 + 0.1 * torch.randn(H)).to(dtype)
    t = {"emb": E.to(DEV), "n.weight": wn.to(DEV)}
    emb = Embedding(EmbeddingSpec(V, H, 12.0, "emb"), t, ctx(dtype))
    head = Head(HeadSpec(V, H, input_divisor=3.0, tied=True, name="lm"), t, emb, ctx(dtype))
    norm = norm_class("rms")(NormSpec("rms", H, 1e-5), t, "n.", ctx(dtype))
    ids = torch.tensor([3, 262, 0, 77], dtype=torch.int32, device=DEV)
    stream = emb.forward(ids)
    h = P.embedding(ids.long().cpu(), E.double(), 12.0)
    assert rel_err(stream.h.cpu().numpy(), h.numpy()) < 1e-6
    rows = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    logits = head.forward(stream, norm, rows)
    assert logits.dtype == torch.float32 and logits.shape == (2, V)
    want = P.linear(P.rms_norm(h[[3, 1]], wn.double(), 1e-5) / 3.0, E.double())
    assert rel_err(logits.cpu().numpy(), want.numpy()) <= TOLS[dtype]


# -- a toy architecture defined outside the framework --------------------------

@dataclass
class ToyConfig:
    width: int
    vocab: int
    decay: float
    layout: List[str]                 # per layer: "ema" or "attn"
    head_dim: int = 16                # of the attention layers (64: the tensor-core attention kernels' shape)

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["vocab"], d["decay"], list(d["layout"]), int(d.get("head_dim", 16)))

    def to_dict(self):
        return {"architectures": ["ToyEmaLM"], "model_type": "toy_ema", "width": self.width, "vocab": self.vocab,
                "decay": self.decay, "layout": self.layout, "head_dim": self.head_dim}


class EmaMixer:
    """y_t = (a * s_{t-1} + (1 - a) * x_t) * w, with the running mean s kept
    per sequence in the cache's fixed-size state (float32)."""

    @staticmethod
    def tensor_specs(spec, prefix):
        from exl3_server_b200.weights import TensorSpec
        return [TensorSpec(prefix + "scale", (spec.width,), init="ones")]

    def __init__(self, spec, tensors, prefix, ctx):
        self.spec = spec
        self.a = float(spec.params["decay"])
        self.w = tensors[prefix + "scale"].float()

    def cache_request(self):
        return None

    def state_request(self):
        from exl3_server_b200.parts import StateRequest
        return StateRequest((self.spec.width,), torch.float32)

    def forward(self, x, batch, kv, state):
        a = self.a
        xf = x.float()
        if batch.max_new == 1:                               # one token per row: safe inside a CUDA graph
            idx = batch.slot_ids.long()
            s = a * state[idx] + (1 - a) * xf
            state.index_copy_(0, idx, s)
            return (s * self.w).to(x.dtype)
        out = torch.empty_like(xf)
        t0 = 0
        for slot, n in zip(batch.host_slots, batch.host_new):
            s = state[slot].clone()
            for i in range(n):
                s = a * s + (1 - a) * xf[t0 + i]
                out[t0 + i] = s * self.w
            state[slot] = s
            t0 += n
        return out.to(x.dtype)


def toy_plan(cfg: ToyConfig):
    from exl3_server_b200.parts import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan,
                                        NormSpec, PositionSpec, ScheduleEntry)
    layers = []
    for i, kind in enumerate(cfg.layout):
        p = f"toy.{i}."
        if kind == "ema":
            mixer = MixerSpec("test_ema", width=cfg.width, params={"decay": cfg.decay})
        else:
            mixer = MixerSpec("attention", width=cfg.width, heads=2, kv_heads=1, head_dim=cfg.head_dim,
                              position=PositionSpec("rope", dims=cfg.head_dim, theta=100.0))
        layers.append(LayerSpec("prenorm", mixer, FeedForwardSpec("swiglu", cfg.width, 2 * cfg.width),
                                NormSpec("rms", cfg.width, 1e-5), NormSpec("rms", cfg.width, 1e-5), 0.5,
                                names={"mixer": p + "mix.", "feed_forward": p + "ff.", "mixer_norm": p + "n1.",
                                       "feed_forward_norm": p + "n2."}))
    n = len(layers)
    # every layer once, then layer 0 again (it has state or a cache of its own for the second run),
    # then the last attention layer once more, reading the keys and values of its first run
    schedule = [ScheduleEntry(i) for i in range(n)] + [ScheduleEntry(0)]
    last_attn = max(i for i, k in enumerate(cfg.layout) if k == "attn")
    schedule.append(ScheduleEntry(last_attn, cache_from=last_attn))
    return ModelPlan("ToyEmaLM", EmbeddingSpec(cfg.vocab, cfg.width, 1.0, "toy.emb"), layers, schedule,
                     NormSpec("rms", cfg.width, 1e-5), "toy.norm.", HeadSpec(cfg.vocab, cfg.width, 1.0, True, "toy.head"),
                     max_positions=0)


def toy_plain_logits(w: Dict[str, torch.Tensor], cfg: ToyConfig, ids: List[int]) -> torch.Tensor:
    """The toy model on one whole sequence, float64, plain loops."""
    w = {k: v.double() for k, v in w.items()}
    L = len(ids)
    h = w["toy.emb"][torch.tensor(ids)]
    n = len(cfg.layout)
    last_attn = max(i for i, k in enumerate(cfg.layout) if k == "attn")
    kv_of = {}
    for si, li in enumerate(list(range(n)) + [0, last_attn]):
        p = f"toy.{li}."
        r = P.rms_norm(h, w[p + "n1.weight"], 1e-5)
        if cfg.layout[li] == "ema":
            s = torch.zeros(cfg.width, dtype=P.F)             # this run of the layer has its own state
            y = torch.empty_like(r)
            for t in range(L):
                s = cfg.decay * s + (1 - cfg.decay) * r[t]
                y[t] = s * w[p + "mix.scale"]
        else:
            hd = cfg.head_dim
            q = P.linear(r, w[p + "mix.q_proj.weight"]).view(L, 2, hd).transpose(0, 1)
            k = P.linear(r, w[p + "mix.k_proj.weight"]).view(L, 1, hd).transpose(0, 1)
            v = P.linear(r, w[p + "mix.v_proj.weight"]).view(L, 1, hd).transpose(0, 1)
            pos = torch.arange(L)
            q, k = P.rope(q, pos, 100.0), P.rope(k, pos, 100.0)
            if si == n + 1:
                k, v = kv_of[last_attn]                         # reads the first run's keys and values
            else:
                kv_of[li] = (k, v)
            y = P.linear(P.attention(q, k, v).transpose(0, 1).reshape(L, -1), w[p + "mix.o_proj.weight"])
        h = h + 0.5 * y
        r = P.rms_norm(h, w[p + "n2.weight"], 1e-5)
        h = h + 0.5 * P.swiglu(r, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
    return P.linear(P.rms_norm(h, w["toy.norm.weight"], 1e-5), w["toy.emb"])


@pytest.mark.parametrize("dtype,head_dim", [("float32", 16), ("bfloat16", 16), ("bfloat16", 64), ("bfloat16", 128)])
def test_toy_architecture_with_state_is_registered_built_and_stepped(tmp_path, dtype, head_dim):
    from exl3_server_b200 import Engine
    from exl3_server_b200.config import register_architecture, unregister_architecture
    from exl3_server_b200.engine.model import plan_manifest
    from exl3_server_b200.parts import register_mixer, unregister
    from exl3_server_b200.weights import write_safetensors
    from exl3_server_b200.weights.random_init import random_tensors
    # heads of 64 or 128 in bfloat16: the last schedule entry, which reads another entry's keys and values, then goes
    # through the tensor-core decode kernel without a cache write of its own
    cfg = ToyConfig(width=32, vocab=50, decay=0.8, layout=["ema", "attn", "ema", "attn"], head_dim=head_dim)
    register_mixer("test_ema", EmaMixer)
    register_architecture(["ToyEmaLM", "toy_ema"], ToyConfig, toy_plan)
    try:
        folder = str(tmp_path)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg.to_dict(), f)
        tensors = dict(random_tensors(plan_manifest(toy_plan(cfg)), seed=3, std=0.15, norm_std=0.1))
        write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
        # two groups of needs: attention layers share one key/value group; ema layers have state only
        assert len(eng.cache.groups) == 1 and len(eng.cache.state) == 3       # layer 0 runs twice: two states
        assert eng.cache.entry_owns == [False, True, False, True, False, False]
        rng = np.random.default_rng(0)
        reqs = {f"r{i}": rng.integers(0, cfg.vocab, n).tolist() for i, n in enumerate([70, 5, 33, 1])}
        want = {rid: toy_plain_logits(tensors, cfg, t).numpy() for rid, t in reqs.items()}
        tol = 1e-5 if dtype == "float32" else 5e-2
        ids = list(reqs)
        traces = [whole_trace(reqs), tail_trace(reqs, 32),
                  batched_trace(reqs, [[ids[0], ids[1], ids[3]], [ids[2], ids[1]]],
                                {ids[0]: 60, ids[1]: 2, ids[2]: 33, ids[3]: 1})]
        for trace in traces:
            got = run_trace(eng, trace)
            for rid in got:
                assert rel_err(got[rid], want[rid]) <= tol, rid
        assert eng.cache.tokens_held() == 0
    finally:
        unregister_architecture(["ToyEmaLM", "toy_ema"])
        unregister("mixer", "test_ema")


# -- more toy parts from outside: a routed feed-forward and another position encoding ----

class RoutedFeedForward:
    """Two experts, each a small gated MLP; a token goes to the expert whose
    router logit is larger (float32 logits) and is scaled by the softmax weight."""

    @staticmethod
    def tensor_specs(spec, prefix):
        from exl3_server_b200.weights import TensorSpec
        out = [TensorSpec(prefix + "router.weight", (2, spec.width))]
        for e in range(2):
            out += [TensorSpec(prefix + f"experts.{e}.gate_proj.weight", (spec.inner, spec.width)),
                    TensorSpec(prefix + f"experts.{e}.up_proj.weight", (spec.inner, spec.width)),
                    TensorSpec(prefix + f"experts.{e}.down_proj.weight", (spec.width, spec.inner))]
        return out

    def __init__(self, spec, tensors, prefix, ctx):
        from exl3_server_b200.parts import FeedForwardSpec, feed_forward_class
        self.router = tensors[prefix + "router.weight"].float()
        dense = feed_forward_class("swiglu")
        self.experts = [dense(FeedForwardSpec("swiglu", spec.width, spec.inner), tensors, prefix + f"experts.{e}.", ctx)
                        for e in range(2)]

    def forward(self, x, batch):
        logits = x.float() @ self.router.T                       # router logits in float32
        w = torch.softmax(logits, dim=-1)
        pick = (logits[:, 1] > logits[:, 0]).to(x.dtype).unsqueeze(1)
        # both experts run on every token (a toy: no grouping), the unpicked one is masked out;
        # no host decision, so the same code runs inside the decode graph
        y0, y1 = self.experts[0].forward(x, batch), self.experts[1].forward(x, batch)
        scale = torch.where(pick.bool(), w[:, 1:2], w[:, 0:1]).to(x.dtype)
        return (y0 * (1 - pick) + y1 * pick) * scale


class HalfSpeedRope:
    """Rotary embedding whose positions advance at half speed (a stand-in for
    scaled variants): same kernel, other frequency table and position scale."""

    def __init__(self, spec, head_dim, ctx):
        self.dims = spec.dims
        d = torch.arange(0, spec.dims // 2, dtype=torch.float64)
        self.inv_freq = (spec.theta ** (-2.0 * d / spec.dims)).float().to(ctx.device)

    def rotate_and_store(self, qkv, batch, kv, heads, kv_heads, head_dim):
        from exl3_server_b200.ops import kernels as K
        K.rope_kv_write(qkv, self.inv_freq, self.dims, 0.5, batch.tok_pos, batch.tok_seq, kv.block_table,
                        kv.k if kv.owns else None, kv.v if kv.owns else None, heads, kv_heads, head_dim,
                        kv.page_size, kv.owns)


class TwoTableEmbedding:
    """An embedding that is not one table gather: a row of the token table plus a row of a small second table
    chosen by the token id modulo its length."""

    @staticmethod
    def tensor_specs(spec):
        from exl3_server_b200.weights import TensorSpec
        return [TensorSpec(spec.name, (spec.vocab, spec.width)),
                TensorSpec(spec.params["second"], (spec.params["classes"], spec.width))]

    def __init__(self, spec, tensors, ctx):
        self.table = tensors[spec.name].to(ctx.dtype)
        self.second = tensors[spec.params["second"]].to(ctx.dtype)
        self.scale = spec.scale

    def forward(self, token_ids):
        from exl3_server_b200.parts import ResidualStream
        ids = token_ids.long()
        return ResidualStream((self.table[ids].float() + self.second[ids % self.second.shape[0]].float()) * self.scale)


class SoftcapHead:
    """A head of its own kind: logits squashed to (-cap, cap) by ``cap * tanh(x / cap)``."""

    @staticmethod
    def tensor_specs(spec):
        from exl3_server_b200.weights import TensorSpec
        return [TensorSpec(spec.name, (spec.vocab, spec.width))]

    def __init__(self, spec, tensors, embedding, ctx):
        from exl3_server_b200.parts.linear import Linear
        self.linear = Linear(tensors[spec.name], None, ctx.dtype)
        self.cap = float(spec.params["cap"])
        self.divisor = spec.input_divisor

    def forward(self, stream, final_norm, rows):
        r = final_norm.add_norm(stream, rows=rows, out_scale=1.0 / self.divisor)
        return self.cap * torch.tanh(self.linear(r, out_dtype=torch.float32) / self.cap)

    def read_bytes(self):
        return self.linear.weight_bytes()


@dataclass
class Toy2Config:
    width: int
    vocab: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["vocab"])

    def to_dict(self):
        return {"architectures": ["ToyRoutedLM"], "width": self.width, "vocab": self.vocab}


def toy2_plan(cfg):
    from exl3_server_b200.parts import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan,
                                        NormSpec, PositionSpec, ScheduleEntry)
    layers = []
    for i in range(2):
        p = f"t.{i}."
        layers.append(LayerSpec(
            "prenorm",
            MixerSpec("attention", width=cfg.width, heads=2, kv_heads=2, head_dim=16,
                      position=PositionSpec("test_half_speed_rope", dims=16, theta=50.0)),
            FeedForwardSpec("test_routed" if i == 1 else "swiglu", cfg.width, 40),
            NormSpec("rms", cfg.width, 1e-5), NormSpec("rms", cfg.width, 1e-5), 1.0,
            names={"mixer": p + "a.", "feed_forward": p + "f.", "mixer_norm": p + "n1.", "feed_forward_norm": p + "n2."}))
    return ModelPlan("ToyRoutedLM",
                     EmbeddingSpec(cfg.vocab, cfg.width, 1.0, "t.emb", kind="test_two_tables",
                                   params={"second": "t.emb2", "classes": 7}),
                     layers, [ScheduleEntry(0), ScheduleEntry(1)], NormSpec("rms", cfg.width, 1e-5), "t.norm.",
                     HeadSpec(cfg.vocab, cfg.width, 1.0, False, "t.head", kind="test_softcap", params={"cap": 2.0}),
                     max_positions=0)


def toy2_plain_logits(w, cfg, ids):
    w = {k: v.double() for k, v in w.items()}
    L = len(ids)
    h = w["t.emb"][torch.tensor(ids)] + w["t.emb2"][torch.tensor(ids) % 7]
    for i in range(2):
        p = f"t.{i}."
        r = P.rms_norm(h, w[p + "n1.weight"], 1e-5)
        q = P.linear(r, w[p + "a.q_proj.weight"]).view(L, 2, 16).transpose(0, 1)
        k = P.linear(r, w[p + "a.k_proj.weight"]).view(L, 2, 16).transpose(0, 1)
        v = P.linear(r, w[p + "a.v_proj.weight"]).view(L, 2, 16).transpose(0, 1)
        pos = torch.arange(L, dtype=P.F) * 0.5                          # half-speed positions
        q, k = P.rope(q, pos, 50.0), P.rope(k, pos, 50.0)
        h = h + P.linear(P.attention(q, k, v).transpose(0, 1).reshape(L, -1), w[p + "a.o_proj.weight"])
        r = P.rms_norm(h, w[p + "n2.weight"], 1e-5)
        if i == 0:
            y = P.swiglu(r, w[p + "f.gate_proj.weight"], w[p + "f.up_proj.weight"], w[p + "f.down_proj.weight"])
        else:
            logits = r @ w[p + "f.router.weight"].T
            sm = torch.softmax(logits, -1)
            y = torch.empty_like(r)
            for t in range(L):
                e = 1 if logits[t, 1] > logits[t, 0] else 0
                y[t] = sm[t, e] * P.swiglu(r[t:t + 1], w[p + f"f.experts.{e}.gate_proj.weight"],
                                           w[p + f"f.experts.{e}.up_proj.weight"],
                                           w[p + f"f.experts.{e}.down_proj.weight"])[0]
        h = h + y
    return 2.0 * torch.tanh(P.linear(P.rms_norm(h, w["t.norm.weight"], 1e-5), w["t.head"]) / 2.0)


def test_toy_routed_feed_forward_and_other_position_encoding(tmp_path):
    """A feed-forward with routing, a position encoding, an embedding and a head of their own kinds, all
    defined here, registered and run through the engine in float32 (where a
    routing decision cannot flip by rounding of the activations)."""
    from exl3_server_b200 import Engine
    from exl3_server_b200.config import register_architecture, unregister_architecture
    from exl3_server_b200.engine.model import plan_manifest
    from exl3_server_b200.parts import (register_embedding, register_feed_forward, register_head, register_position,
                                        unregister)
    from exl3_server_b200.weights import write_safetensors
    from exl3_server_b200.weights.random_init import random_tensors
    cfg = Toy2Config(width=32, vocab=40)
    register_feed_forward("test_routed", RoutedFeedForward)
    register_position("test_half_speed_rope", HalfSpeedRope)
    register_embedding("test_two_tables", TwoTableEmbedding)
    register_head("test_softcap", SoftcapHead)
    register_architecture(["ToyRoutedLM"], Toy2Config, toy2_plan)
    try:
        folder = str(tmp_path)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg.to_dict(), f)
        tensors = dict(random_tensors(plan_manifest(toy2_plan(cfg)), seed=5, std=0.2, norm_std=0.1))
        write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=512)
        rng = np.random.default_rng(1)
        reqs = {f"r{i}": rng.integers(0, cfg.vocab, n).tolist() for i, n in enumerate([50, 7, 33])}
        want = {rid: toy2_plain_logits(tensors, cfg, t).numpy() for rid, t in reqs.items()}
        ids = list(reqs)
        for trace in (whole_trace(reqs), tail_trace(reqs, 32),
                      batched_trace(reqs, [ids], {ids[0]: 40, ids[1]: 1, ids[2]: 33})):
            got = run_trace(eng, trace)
            for rid in got:
                assert rel_err(got[rid], want[rid]) <= 2e-5, rid
        # both experts were used, so the routing was exercised
        r = torch.randn(64, 32, dtype=torch.float64) @ tensors["t.1.f.router.weight"].double().T
        assert 0 < int((r[:, 1] > r[:, 0]).sum()) < 64
    finally:
        unregister_architecture(["ToyRoutedLM"])
        unregister("feed_forward", "test_routed")
        unregister("position", "test_half_speed_rope")
        unregister("embedding", "test_two_tables")
        unregister("head", "test_softcap")


# -- a mixer whose keys and values differ in width (its cache group has pools of two shapes) ----

class WideValueMixer:
    """Causal attention with narrow keys (16 per head) and wide values (32 per head), no position encoding,
    written with tensor operations only, so that the same code runs inside the recorded decode step."""

    HEADS, DK, DV = 2, 16, 32

    @classmethod
    def tensor_specs(cls, spec, prefix):
        from exl3_server_b200.weights import TensorSpec
        h = cls.HEADS
        return [TensorSpec(prefix + "wq", (h * cls.DK, spec.width)), TensorSpec(prefix + "wk", (h * cls.DK, spec.width)),
                TensorSpec(prefix + "wv", (h * cls.DV, spec.width)), TensorSpec(prefix + "wo", (spec.width, h * cls.DV))]

    def __init__(self, spec, tensors, prefix, ctx):
        self.w = {n: tensors[prefix + n].float() for n in ("wq", "wk", "wv", "wo")}

    def cache_request(self):
        from exl3_server_b200.parts import KVRequest
        return KVRequest(self.HEADS, self.DK, 0, value_dim=self.DV)

    def state_request(self):
        return None

    def forward(self, x, batch, kv, state):
        T, H, P = x.shape[0], self.HEADS, kv.page_size
        xf = x.float()
        q = (xf @ self.w["wq"].T).view(T, H, self.DK)
        k = (xf @ self.w["wk"].T).view(T, H, self.DK)
        v = (xf @ self.w["wv"].T).view(T, H, self.DV)
        rows, pos = batch.tok_seq.long(), batch.tok_pos.long()
        table = kv.block_table.long()
        page = table[rows, pos // P]
        kv.k[page, :, pos % P] = k.to(kv.k.dtype)
        kv.v[page, :, pos % P] = v.to(kv.v.dtype)
        mine = table[rows]                                           # [T, pages]; -1 beyond a row's pages
        keys = kv.k[mine].permute(0, 2, 1, 3, 4).reshape(T, H, -1, self.DK).float()
        vals = kv.v[mine].permute(0, 2, 1, 3, 4).reshape(T, H, -1, self.DV).float()
        s = torch.einsum("thd,thkd->thk", q, keys) / math.sqrt(self.DK)
        later = torch.arange(keys.shape[2], device=x.device)[None, :] > pos[:, None]
        s = s.masked_fill(later[:, None, :], float("-inf"))
        o = torch.einsum("thk,thkd->thd", torch.softmax(s, dim=-1), vals)
        return (o.reshape(T, -1) @ self.w["wo"].T).to(x.dtype)


@dataclass
class Toy3Config:
    width: int
    vocab: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["vocab"])

    def to_dict(self):
        return {"architectures": ["ToyWideValueLM"], "width": self.width, "vocab": self.vocab}


def toy3_plan(cfg):
    from exl3_server_b200.parts import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan,
                                        NormSpec, ScheduleEntry)
    layers = [LayerSpec("prenorm", MixerSpec("test_wide_value", width=cfg.width),
                        FeedForwardSpec("swiglu", cfg.width, 48), NormSpec("rms", cfg.width, 1e-5),
                        NormSpec("rms", cfg.width, 1e-5), 1.0,
                        names={"mixer": f"w.{i}.m.", "feed_forward": f"w.{i}.f.", "mixer_norm": f"w.{i}.n1.",
                               "feed_forward_norm": f"w.{i}.n2."}) for i in range(2)]
    return ModelPlan("ToyWideValueLM", EmbeddingSpec(cfg.vocab, cfg.width, 1.0, "w.emb"), layers,
                     [ScheduleEntry(0), ScheduleEntry(1)], NormSpec("rms", cfg.width, 1e-5), "w.norm.",
                     HeadSpec(cfg.vocab, cfg.width, 1.0, None, "w.head"), max_positions=0)


def toy3_plain_logits(w, cfg, ids):
    w = {k: v.double() for k, v in w.items()}
    L, H, DK, DV = len(ids), WideValueMixer.HEADS, WideValueMixer.DK, WideValueMixer.DV
    h = w["w.emb"][torch.tensor(ids)]
    for i in range(2):
        p = f"w.{i}."
        r = P.rms_norm(h, w[p + "n1.weight"], 1e-5)
        q = P.linear(r, w[p + "m.wq"]).view(L, H, DK).transpose(0, 1)
        k = P.linear(r, w[p + "m.wk"]).view(L, H, DK).transpose(0, 1)
        v = P.linear(r, w[p + "m.wv"]).view(L, H, DV).transpose(0, 1)
        s = (q @ k.transpose(1, 2)) / math.sqrt(DK)
        s = s.masked_fill(torch.arange(L)[None, :] > torch.arange(L)[:, None], float("-inf"))
        o = (torch.softmax(s, dim=-1) @ v).transpose(0, 1).reshape(L, -1)
        h = h + P.linear(o, w[p + "m.wo"])
        r = P.rms_norm(h, w[p + "n2.weight"], 1e-5)
        h = h + P.swiglu(r, w[p + "f.gate_proj.weight"], w[p + "f.up_proj.weight"], w[p + "f.down_proj.weight"])
    return P.linear(P.rms_norm(h, w["w.norm.weight"], 1e-5), w["w.emb"])     # no head tensor: tied


def test_toy_mixer_with_keys_and_values_of_different_widths(tmp_path):
    """A mixer from outside whose cache holds 16 numbers per key and 32 per value: the cache makes a group with two
    pool shapes for it, and the step function, the decode graphs and slot reuse work unchanged.  The head's tie is
    left to the checkpoint (no head tensor: tied)."""
    from exl3_server_b200 import Engine
    from exl3_server_b200.config import register_architecture, unregister_architecture
    from exl3_server_b200.engine.model import plan_manifest
    from exl3_server_b200.parts import register_mixer, unregister
    from exl3_server_b200.weights import write_safetensors
    from exl3_server_b200.weights.random_init import random_tensors
    cfg = Toy3Config(width=32, vocab=40)
    register_mixer("test_wide_value", WideValueMixer)
    register_architecture(["ToyWideValueLM"], Toy3Config, toy3_plan)
    try:
        folder = str(tmp_path)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg.to_dict(), f)
        tensors = dict(random_tensors(plan_manifest(toy3_plan(cfg)), seed=8, std=0.2, norm_std=0.1))
        assert "w.head" not in tensors                                  # optional and not written: the head is tied
        write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024)
        group = eng.cache.groups[0]
        assert group.k.shape[-1] == 16 and group.v.shape[-1] == 32 and eng.model.head.tied
        rng = np.random.default_rng(2)
        reqs = {f"r{i}": rng.integers(0, cfg.vocab, n).tolist() for i, n in enumerate([70, 5, 130, 1])}
        want = {rid: toy3_plain_logits(tensors, cfg, t).numpy() for rid, t in reqs.items()}
        ids = list(reqs)
        for trace in (whole_trace(reqs), tail_trace(reqs, 32),
                      batched_trace(reqs, [[ids[0], ids[1], ids[3]], [ids[2], ids[1]]],
                                    {ids[0]: 60, ids[1]: 2, ids[2]: 100, ids[3]: 1})):
            got = run_trace(eng, trace)
            for rid in got:
                assert rel_err(got[rid], want[rid]) <= 2e-5, rid
        assert eng.cache.tokens_held() == 0
    finally:
        unregister_architecture(["ToyWideValueLM"])
        unregister("mixer", "test_wide_value")
