"""The plain implementation checked against hand-computed cases, so that the
oracle itself rests on more than its own code."""
import math

import torch

import plain_llama as P


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=P.F)
    w = torch.tensor([2.0, 0.5], dtype=P.F)
    inv = 1.0 / math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(P.rms_norm(x, w, 1e-6), torch.tensor([[3 * inv * 2, 4 * inv * 0.5]], dtype=P.F))


def test_rope_is_a_rotation_of_half_split_pairs():
    hd = 4
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0], [1.0, 2.0, 3.0, 4.0]]], dtype=P.F)   # one head, positions 0 and 3
    y = P.rope(x, torch.tensor([0, 3]), theta=100.0)
    assert torch.allclose(y[0, 0], x[0, 0])                    # position 0: identity
    f = [1.0, 100.0 ** (-2 / 4)]
    for d in range(2):
        a = 3 * f[d]
        assert math.isclose(float(y[0, 1, d]), x[0, 1, d] * math.cos(a) - x[0, 1, d + 2] * math.sin(a))
        assert math.isclose(float(y[0, 1, d + 2]), x[0, 1, d + 2] * math.cos(a) + x[0, 1, d] * math.sin(a))
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q = torch.randn(4, 6, 8, dtype=P.F)
    k = torch.randn(2, 6, 8, dtype=P.F)
    v = torch.randn(2, 6, 8, dtype=P.F)
    o = P.attention(q, k, v)
    assert torch.allclose(o[:, 0], v.repeat_interleave(2, dim=0)[:, 0])      # first token sees itself only
    # head 3 reads kv head 1; position 2 by hand
    s = (q[3, 2] @ k[1, :3].T) / math.sqrt(8)
    want = torch.softmax(s, -1) @ v[1, :3]
    assert torch.allclose(o[3, 2], want)
    # changing a later key changes nothing earlier
    k2 = k.clone()
    k2[:, 5] += 1.0
    assert torch.allclose(P.attention(q, k2, v)[:, :5], o[:, :5])
    # a window of 2 keys
    ow = P.attention(q, k, v, window=2)
    s = (q[0, 4] @ k[0, 3:5].T) / math.sqrt(8)
    assert torch.allclose(ow[0, 4], torch.softmax(s, -1) @ v[0, 3:5])


def test_swiglu_by_hand():
    r = torch.tensor([[1.0, -2.0]], dtype=P.F)
    wg = torch.tensor([[1.0, 0.0]], dtype=P.F)
    wu = torch.tensor([[0.0, 1.0]], dtype=P.F)
    wd = torch.tensor([[2.0], [3.0]], dtype=P.F)
    g, u = 1.0, -2.0
    a = g / (1 + math.exp(-g)) * u
    assert torch.allclose(P.swiglu(r, wg, wu, wd), torch.tensor([[2 * a, 3 * a]], dtype=P.F))


def test_forward_prefix_property(model_folders):
    """Logits at a position depend only on the tokens up to it."""
    pm = P.PlainModel(model_folders["C"])
    ids = list(range(3, 60))
    full = pm.logits(ids)
    assert torch.allclose(pm.logits(ids[:31]), full[:31], atol=1e-12)


def test_rotary_table_keeps_what_float32_loses():
    """The kernels' frequency table: two float32 rows whose sum is the float64 frequency to about 1e-15 of it, so
    that position * frequency keeps its accuracy at large positions."""
    import torch
    from exl3_server_b200.ops.kernels import rotary_table
    f = torch.pow(torch.tensor(500000.0, dtype=torch.float64), -2.0 * torch.arange(0, 64, dtype=torch.float64) / 128)
    t = rotary_table(f)
    assert t.dtype == torch.float32 and tuple(t.shape) == (2, 64) and t.is_contiguous()
    back = t[0].double() + t[1].double()
    assert float(((back - f).abs() / f).max()) < 1e-14
    assert float(((t[0].double() - f).abs() / f).max()) > 1e-9          # the first row alone is float32
    pos = 150001.0
    assert float((pos * back - pos * f).abs().max()) < 1e-9
