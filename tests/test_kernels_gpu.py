"""Each CUDA kernel alone against a plain float32/float64 torch computation of
the same operation, at sizes other than the engine tests use (widths and
vocabularies that are no power of two, head sizes in steps of 16, grouped
heads, windows, ragged batches)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def K():
    from exl3_server_b200.ops import kernels
    return kernels


def close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / max(1e-30, float(want.abs().max())))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.0e}"


TOL = {torch.float32: 2e-6, torch.bfloat16: 1.2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    torch.manual_seed(0)
    table = torch.randn(1003, 72, device=DEV).to(dtype)
    ids = torch.tensor([0, 1002, 5, 5, 77], dtype=torch.int32, device=DEV)
    out = K().embed(ids, table, 12.0)
    assert out.dtype == torch.float32
    close(out, table.float()[ids.long()] * 12.0, 1e-7, "embed")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [72, 2304, 1000])
def test_add_rmsnorm(dtype, H):
    torch.manual_seed(1)
    T = 7
    h = torch.randn(T, H, device=DEV)
    y = torch.randn(T, H, device=DEV).to(dtype)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(dtype)
    h0 = h.clone()
    out = K().add_rmsnorm(h, y, 0.37, w, 1e-5, dtype, out_scale=0.5)
    hn = h0.double() + y.double() * 0.37
    close(h, hn, 1e-6, "residual")
    want = hn * torch.rsqrt((hn * hn).mean(-1, keepdim=True) + 1e-5) * w.double() * 0.5
    close(out, want, TOL[dtype], "norm")
    # without a pending output, on listed rows only, float32 weight in the bfloat16 path
    rows = torch.tensor([6, 2], dtype=torch.int32, device=DEV)
    h1 = h.clone()
    out = K().add_rmsnorm(h, None, 1.0, w.float(), 1e-5, dtype, rows=rows)
    assert torch.equal(h, h1) and out.shape == (2, H)
    hh = h1.double()[[6, 2]]
    close(out, hh * torch.rsqrt((hh * hh).mean(-1, keepdim=True) + 1e-5) * w.double(), TOL[dtype], "rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [173, 176, 5760])
def test_silu_mul(dtype, I):
    torch.manual_seed(2)
    gu = (3 * torch.randn(5, 2 * I, device=DEV)).to(dtype)
    g, u = gu.double()[:, :I], gu.double()[:, I:]
    close(K().silu_mul(gu), g * torch.sigmoid(g) * u, TOL[dtype], "silu_mul")
    if I % 8 == 0:
        n = I // 8
        inter = torch.stack([gu[:, :I].reshape(5, n, 8), gu[:, I:].reshape(5, n, 8)], dim=2).reshape(5, 2 * I)
        close(K().silu_mul(inter.contiguous(), interleave=8), g * torch.sigmoid(g) * u, TOL[dtype], "interleaved")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,Kd", [(1, 50, 24), (5, 263, 96), (70, 130, 200), (3, 64, 7), (17, 33, 65)])
def test_gemm_simt(dtype, M, N, Kd):
    torch.manual_seed(3)
    x = torch.randn(M, Kd, device=DEV).to(dtype)
    w = torch.randn(N, Kd, device=DEV).to(dtype)
    b = torch.randn(N, device=DEV).to(dtype)
    want = x.double() @ w.double().T + b.double()
    close(K().gemm_simt(x, w, b, dtype), want, TOL[dtype], "gemm")
    if dtype == torch.bfloat16:
        close(K().gemm_simt(x, w, None, torch.float32), x.double() @ w.double().T, 2e-6, "gemm f32 out")


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    torch.manual_seed(4)
    x = torch.randn(70, 300, device=DEV)
    w = torch.randn(90, 300, device=DEV)
    full = K().gemm_simt(x, w, None, torch.float32)
    for r in (0, 13, 69):
        assert torch.equal(K().gemm_simt(x[r:r + 1].contiguous(), w, None, torch.float32)[0], full[r])


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,Kd", [(2304, 2304), (263, 96), (50, 40), (1000, 5768), (16, 8)])
def test_gemv_bf16(M, N, Kd):
    torch.manual_seed(5)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    want = x.double() @ w.double().T
    close(K().gemv_bf16(x, w, None, torch.float32), want, 2e-6, "gemv f32 out")
    close(K().gemv_bf16(x, w, b, torch.bfloat16), want + b.double(), TOL[torch.bfloat16], "gemv bf16 out")
    # a row's result does not depend on the other rows
    one = K().gemv_bf16(x[M - 1:].contiguous(), w, None, torch.float32)
    assert torch.equal(one[0], K().gemv_bf16(x, w, None, torch.float32)[M - 1])


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,Kd", [(176, 64), (5760, 2304), (200, 96)])
def test_gemv_gated_and_interleaved_silu(M, I, Kd):
    torch.manual_seed(9)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    wg = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    wu = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    bg, bu = torch.randn(I, device=DEV).bfloat16(), torch.randn(I, device=DEV).bfloat16()
    n = I // 8
    w = torch.stack([wg.view(n, 8, Kd), wu.view(n, 8, Kd)], dim=1).reshape(2 * I, Kd).contiguous()
    b = torch.stack([bg.view(n, 8), bu.view(n, 8)], dim=1).reshape(-1).contiguous()
    g = x.double() @ wg.double().T + bg.double()
    u = x.double() @ wu.double().T + bu.double()
    want = g * torch.sigmoid(g) * u
    close(K().gemv_bf16(x, w, b, torch.bfloat16, gated=True), want, TOL[torch.bfloat16], "gated gemv")
    close(K().gemv_bf16(x, w, b, torch.float32, gated=True), want, 2e-6, "gated gemv f32 out")
    gu = K().gemv_bf16(x, w, b, torch.float32)
    close(K().silu_mul(gu, interleave=8), want, 2e-6, "interleaved silu_mul")


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (128, 256, 192), (200, 512, 2304), (77, 264, 72), (1, 8, 8),
                                    (2048, 2304, 5760), (300, 6912, 2304)])
def test_gemm_tc(M, N, Kd):
    torch.manual_seed(10)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    want = x.double() @ w.double().T
    close(K().gemm_tc(x, w, None), want, TOL[torch.bfloat16], "gemm_tc")
    close(K().gemm_tc(x, w, b), want + b.double(), TOL[torch.bfloat16], "gemm_tc + bias")
    torch.cuda.synchronize()
    assert K().gemm_tc_status() == 0


@pytest.mark.parametrize("M", [17, 300, 2048])
@pytest.mark.parametrize("I,Kd", [(176, 64), (5760, 2304), (200, 96)])
def test_gemm_tc_gated(M, I, Kd):
    torch.manual_seed(11)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    wg = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    wu = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    bg, bu = torch.randn(I, device=DEV).bfloat16(), torch.randn(I, device=DEV).bfloat16()
    n = I // 8
    w = torch.stack([wg.view(n, 8, Kd), wu.view(n, 8, Kd)], dim=1).reshape(2 * I, Kd).contiguous()
    b = torch.stack([bg.view(n, 8), bu.view(n, 8)], dim=1).reshape(-1).contiguous()
    g = x.double() @ wg.double().T + bg.double()
    u = x.double() @ wu.double().T + bu.double()
    close(K().gemm_tc(x, w, b, gated=True), g * torch.sigmoid(g) * u, TOL[torch.bfloat16], "gated gemm_tc")
    torch.cuda.synchronize()
    assert K().gemm_tc_status() == 0


def test_gemm_tc_waits_are_bounded():
    """A wait that nothing satisfies runs out, the kernel records a code and
    returns; the context stays usable and the next GEMM is right."""
    torch.cuda.synchronize()
    assert K().gemm_tc_status() == 0
    K().gemm_tc_wait_selftest()
    torch.cuda.synchronize()
    assert K().gemm_tc_status() == 9
    assert K().gemm_tc_status() == 0                     # reading clears it
    x = torch.randn(130, 64, device=DEV).bfloat16()
    w = torch.randn(24, 64, device=DEV).bfloat16()
    close(K().gemm_tc(x, w, None), x.double() @ w.double().T, TOL[torch.bfloat16], "gemm_tc after a timed-out wait")


@pytest.mark.parametrize("M", [1, 5, 8, 16])
@pytest.mark.parametrize("N,Kd", [(2304, 2304), (2304, 5760), (263, 96), (50, 40), (136, 208)])
@pytest.mark.parametrize("norm_dtype", [torch.bfloat16, torch.float32])
def test_gemv_folds_into_the_residual_and_prepares_the_norm(M, N, Kd, norm_dtype):
    """The producing side of a norm that is no kernel of its own: h += y * rho, x_raw = h * w, sums of squares."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    nw = (1.0 + 0.2 * torch.randn(N, generator=g)).to(norm_dtype).to(DEV)
    h0 = torch.randn(M, N, generator=g).to(DEV)
    rho, eps = 0.37, 1e-5
    for bias in (None, b):
        h = h0.clone()
        x_raw, ss = K().gemv_bf16_normed(x, w, bias, torch.bfloat16, resid=(h, rho, nw))
        y = K().gemv_bf16(x, w, bias, torch.bfloat16)       # what the plain kernel stores
        want_h = h0.double() + y.double() * rho
        close(h, want_h, 2e-6, "residual")
        close(x_raw, want_h * nw.double(), 6e-3, "residual times the norm weight")
        assert ss.shape == (16, (N + 15) // 16)
        close(ss[:M].sum(1), (want_h * want_h).sum(1), 1e-5, "sums of squares")
        if M < 16:
            assert float(ss[M:].abs().max()) == 0.0
        # the consuming side: a second projection over the norm's output, against the two kernels in turn
        N2 = 176
        w2 = (torch.randn(N2, N, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
        b2 = torch.randn(N2, generator=g).to(torch.bfloat16).to(DEV)
        if N % 8 == 0:
            h2 = h0.clone()
            r = K().add_rmsnorm(h2, y, rho, nw, eps, torch.bfloat16)
            for bias2 in (None, b2):
                want = r.double() @ w2.double().T + (0 if bias2 is None else bias2.double())
                got = K().gemv_bf16_normed(x_raw, w2, bias2, torch.float32, scale=(ss, eps, float(N)))
                close(got, want, 1e-2, "second projection")
            wg = torch.stack([w2[:N2 // 2].view(-1, 8, N), w2[N2 // 2:].view(-1, 8, N)], dim=1).reshape(N2, N).contiguous()
            got = K().gemv_bf16_normed(x_raw, wg, None, torch.bfloat16, gated=True, scale=(ss, eps, float(N)))
            gate, up = r.double() @ w2[:N2 // 2].double().T, r.double() @ w2[N2 // 2:].double().T
            close(got, torch.nn.functional.silu(gate) * up, 1.5e-2, "gated second projection")


@pytest.mark.parametrize("M", [1, 17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("N,Kd", [(2304, 2304), (6912, 2304), (263, 96), (50, 40), (1000, 5768), (16, 8), (136, 208)])
def test_gemm_skinny(M, N, Kd):
    """The weights as the 128-row tensor-core operand, K cut over the blocks of a cluster: every number of cuts,
    sizes that are no multiple of a tile, and a row's result independent of its batch."""
    torch.manual_seed(12)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    want = x.double() @ w.double().T
    # float32 out of bfloat16 operands: tcgen05.mma adds an instruction's products with fewer guard bits than a
    # chain of float32 FMAs keeps (3e-6 of the largest value measured at K = 2304, against 7e-7 for mma.sync),
    # far below the 4e-3 that rounding the operands to bfloat16 costs
    F32 = 1e-5
    auto = K().gemm_skinny(x, w, None, torch.float32)
    close(auto, want, F32, "skinny f32 out")
    close(K().gemm_skinny(x, w, b, torch.bfloat16), want + b.double(), TOL[torch.bfloat16], "skinny bf16 out + bias")
    ksteps = (Kd + 63) // 64
    chosen = K().gemm_skinny_split(N, Kd)
    assert 1 <= chosen <= min(8, ksteps)
    for split in range(1, min(8, ksteps) + 1):
        got = K().gemm_skinny(x, w, None, torch.float32, split=split, tiles=1)
        close(got, want, F32, f"skinny with {split} cuts")
        # two tiles of w per block read x once for both: the same numbers bit for bit
        assert torch.equal(K().gemm_skinny(x, w, None, torch.float32, split=split, tiles=2), got)
        if split == chosen:
            assert torch.equal(got, auto)
    # a row's result does not depend on the other rows, nor on how many there are
    one = K().gemm_skinny(x[M - 1:].contiguous(), w, None, torch.float32)
    assert torch.equal(one[0], auto[M - 1])
    torch.cuda.synchronize()
    assert K().gemm_skinny_status() == 0


@pytest.mark.parametrize("M", [17, 40, 64])
@pytest.mark.parametrize("I,Kd", [(176, 64), (5760, 2304), (200, 96)])
def test_gemm_skinny_gated(M, I, Kd):
    torch.manual_seed(13)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    wg = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    wu = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    bg, bu = torch.randn(I, device=DEV).bfloat16(), torch.randn(I, device=DEV).bfloat16()
    n = I // 8
    w = torch.stack([wg.view(n, 8, Kd), wu.view(n, 8, Kd)], dim=1).reshape(2 * I, Kd).contiguous()
    b = torch.stack([bg.view(n, 8), bu.view(n, 8)], dim=1).reshape(-1).contiguous()
    g = x.double() @ wg.double().T + bg.double()
    u = x.double() @ wu.double().T + bu.double()
    want = g * torch.sigmoid(g) * u
    close(K().gemm_skinny(x, w, b, torch.bfloat16, gated=True), want, TOL[torch.bfloat16], "gated skinny")
    close(K().gemm_skinny(x, w, b, torch.float32, gated=True), want, 1e-5, "gated skinny f32 out")
    assert torch.equal(K().gemm_skinny(x, w, b, torch.bfloat16, gated=True, tiles=2),
                       K().gemm_skinny(x, w, b, torch.bfloat16, gated=True, tiles=1))
    torch.cuda.synchronize()
    assert K().gemm_skinny_status() == 0


@pytest.mark.parametrize("M", [17, 33, 64])
@pytest.mark.parametrize("N,Kd", [(2304, 2304), (2304, 5760), (263, 96), (50, 40), (136, 208)])
@pytest.mark.parametrize("norm_dtype", [torch.bfloat16, torch.float32])
def test_gemm_skinny_folds_into_the_residual_and_prepares_the_norm(M, N, Kd, norm_dtype):
    """Both sides of a norm that is no kernel of its own, for more rows than the GEMV takes."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    nw = (1.0 + 0.2 * torch.randn(N, generator=g)).to(norm_dtype).to(DEV)
    h0 = torch.randn(M, N, generator=g).to(DEV)
    rho, eps = 0.37, 1e-5
    for bias in (None, b):
        h = h0.clone()
        x_raw, ss = K().gemm_skinny(x, w, bias, torch.bfloat16, resid=(h, rho, nw))
        y = K().gemm_skinny(x, w, bias, torch.bfloat16)      # what the plain epilogue stores
        want_h = h0.double() + y.double() * rho
        close(h, want_h, 2e-6, "residual")
        close(x_raw, want_h * nw.double(), 6e-3, "residual times the norm weight")
        assert ss.shape == (M, (N + 15) // 16)
        close(ss.sum(1), (want_h * want_h).sum(1), 1e-5, "sums of squares")
        N2 = 176
        w2 = (torch.randn(N2, N, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
        b2 = torch.randn(N2, generator=g).to(torch.bfloat16).to(DEV)
        if N % 8 == 0:
            h2 = h0.clone()
            r = K().add_rmsnorm(h2, y, rho, nw, eps, torch.bfloat16)
            for bias2 in (None, b2):
                want = r.double() @ w2.double().T + (0 if bias2 is None else bias2.double())
                got = K().gemm_skinny(x_raw, w2, bias2, torch.float32, scale=(ss, eps, float(N)))
                close(got, want, 1e-2, "second projection")
            wg = torch.stack([w2[:N2 // 2].view(-1, 8, N), w2[N2 // 2:].view(-1, 8, N)], dim=1).reshape(N2, N).contiguous()
            got = K().gemm_skinny(x_raw, wg, None, torch.bfloat16, gated=True, scale=(ss, eps, float(N)))
            gate, up = r.double() @ w2[:N2 // 2].double().T, r.double() @ w2[N2 // 2:].double().T
            close(got, torch.nn.functional.silu(gate) * up, 1.5e-2, "gated second projection")
    torch.cuda.synchronize()
    assert K().gemm_skinny_status() == 0


# Sizes for the paired GEMM: one tile; ragged in M, N and K; one row more than a pair's even block holds; fewer
# columns than a staging tile; more tiles than the GPU has pairs (several per pair, both accumulators in turn).
PAIR_SIZES = [(256, 256, 64), (300, 520, 264), (129, 16, 8), (65, 4608, 128), (1000, 1000, 1000), (2048, 2304, 2304),
              (5000, 2304, 72)]


@pytest.mark.parametrize("M,N,Kd", PAIR_SIZES)
def test_gemm_pair(M, N, Kd):
    """Two blocks of a cluster as one tensor core (tcgen05.mma.cta_group::2): plain, with a bias, with a norm's row
    factors, and a row's result independent of the other rows."""
    torch.manual_seed(14)
    x = (torch.randn(M, Kd, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    want = x.double() @ w.double().T
    got = K().gemm_pair(x, w, None)
    close(got, want, TOL[torch.bfloat16], "pair")
    close(K().gemm_pair(x, w, b), want + b.double(), TOL[torch.bfloat16], "pair + bias")
    width, eps = 77.0, 1e-5
    ss = torch.rand(M + 3, 5, device=DEV) * 40 + 1
    k = torch.rsqrt(ss[:M].sum(1) / width + eps).double()
    close(K().gemm_pair(x, w, b, scale=(ss, eps, width)), want * k[:, None] + b.double(), TOL[torch.bfloat16],
          "pair with row factors")
    # the last rows alone: other tiles, another place in their tile, the same numbers
    tail = K().gemm_pair(x[M - 40:].contiguous(), w, None)
    assert torch.equal(tail, got[M - 40:])
    torch.cuda.synchronize()
    assert K().gemm_pair_status() == 0


@pytest.mark.parametrize("M,I,Kd", [(256, 128, 64), (300, 264, 264), (129, 8, 8), (2048, 5760, 2304), (700, 1000, 520)])
def test_gemm_pair_gated(M, I, Kd):
    torch.manual_seed(15)
    x = (torch.randn(M, Kd, device=DEV) * 0.5).bfloat16()
    wg = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    wu = (torch.randn(I, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    bg, bu = torch.randn(I, device=DEV).bfloat16(), torch.randn(I, device=DEV).bfloat16()
    n = I // 8
    w = torch.stack([wg.view(n, 8, Kd), wu.view(n, 8, Kd)], dim=1).reshape(2 * I, Kd).contiguous()
    b = torch.stack([bg.view(n, 8), bu.view(n, 8)], dim=1).reshape(-1).contiguous()
    g = x.double() @ wg.double().T + bg.double()
    u = x.double() @ wu.double().T + bu.double()
    close(K().gemm_pair(x, w, b, gated=True), g * torch.sigmoid(g) * u, TOL[torch.bfloat16], "gated pair")
    # against the one-block kernel with the same epilogue
    close(K().gemm_pair(x, w, b, gated=True), K().gemm_tc(x, w, b, gated=True).double(), TOL[torch.bfloat16], "pair and one block")
    torch.cuda.synchronize()
    assert K().gemm_pair_status() == 0


@pytest.mark.parametrize("M,N,Kd", PAIR_SIZES)
@pytest.mark.parametrize("norm_dtype", [torch.bfloat16, torch.float32])
def test_gemm_pair_folds_into_the_residual_and_prepares_the_norm(M, N, Kd, norm_dtype):
    """The residual goes into the accumulator before the products and comes out with them added: h in place,
    h times the norm's weight, and the row sums of h squared per tile of 256 columns; then both pieces into the
    next projection.  With 5,000 rows a pair has several tiles and brings the residual of a later tile in while
    the tensor core works on an earlier one."""
    g = torch.Generator().manual_seed(M + N)
    x = (torch.randn(M, Kd, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    nw = (1.0 + 0.2 * torch.randn(N, generator=g)).to(norm_dtype).to(DEV)
    h0 = (torch.randn(M, N, generator=g) * 3).to(DEV)
    rho, eps = 0.37, 1e-5
    width = 77.0
    ss_in = (torch.rand(M, 3, generator=g) * 40 + 1).to(DEV)
    k = torch.rsqrt(ss_in.sum(1) / width + eps).double()
    for bias, scale in ((None, None), (b, None), (b, (ss_in, eps, width))):
        h = h0.clone()
        x_raw, ss = K().gemm_pair(x, w, bias, scale=scale, resid=(h, rho, nw))
        y = x.double() @ w.double().T * (1.0 if scale is None else k[:, None]) + (0 if bias is None else bias.double())
        want_h = h0.double() + y * rho
        # the products are added to h inside the tensor core: 1e-5 of the largest h (fewer guard bits than a chain
        # of float32 FMAs), against the 2e-3 that rounding the product to bfloat16 first would cost
        close(h, want_h, 2e-5, "residual")
        close(x_raw, want_h * nw.double(), 6e-3, "residual times the norm weight")
        assert ss.shape == (M, (N + 255) // 256)
        close(ss.sum(1), (want_h * want_h).sum(1), 2e-5, "sums of squares")
    # the pieces feed the next projection as the norm's output would
    if N % 8 == 0:
        N2 = 176
        w2 = (torch.randn(N2, N, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
        r = (h.double() * torch.rsqrt((h.double() ** 2).mean(1, keepdim=True) + eps) * nw.double())
        got = K().gemm_pair(x_raw, w2, None, scale=(ss, eps, float(N)))
        close(got, r @ w2.double().T, 1e-2, "second projection")
    torch.cuda.synchronize()
    assert K().gemm_pair_status() == 0


@pytest.mark.parametrize("lens,starts", [([2048], [0]),               # one prompt: every warp's rows are one page's places
                                         ([300, 64, 1, 515], [0, 0, 0, 0]),  # sequences that start anywhere in a tile
                                         ([200, 96], [64, 1000])])           # prompts that go on from earlier tokens
@pytest.mark.parametrize("nh,nkv", [(4, 4), (6, 2), (3, 1)])
@pytest.mark.parametrize("rot", [64, 0])
def test_gemm_pair_rotates_and_writes_the_cache(lens, starts, nh, nkv, rot):
    """The q/k/v projection with the position step in its epilogue, against the projection followed by the
    kernel of that step: the same queries, and the same keys and values at every token's place in the cache
    (and nothing written anywhere else)."""
    torch.manual_seed(16)
    hd, page, Kd = 64, 64, 136
    T = sum(lens)
    N = (nh + 2 * nkv) * hd
    x = (torch.randn(T, Kd, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    need = [(s0 + n + page - 1) // page for s0, n in zip(starts, lens)]
    n_pages = sum(need) + 3
    perm = torch.randperm(n_pages).tolist()
    table = torch.full((len(lens), max(need)), -1, dtype=torch.int32)
    at = 0
    for i, n in enumerate(need):
        table[i, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    table = table.to(DEV)
    tok_pos = torch.cat([torch.arange(s0, s0 + n) for s0, n in zip(starts, lens)]).to(torch.int32).to(DEV)
    tok_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32).to(DEV)
    inv_freq = K().rotary_table(torch.pow(torch.tensor(10000.0, dtype=torch.float64),
                                          -2.0 * torch.arange(0, hd // 2, dtype=torch.float64) / hd)).to(DEV)
    junk_k = torch.randn(n_pages, nkv, page, hd, device=DEV).bfloat16()
    junk_v = torch.randn(n_pages, nkv, page, hd, device=DEV).bfloat16()
    # the separate steps
    want = K().gemm_pair(x, w, b)
    k1, v1 = junk_k.clone(), junk_v.clone()
    K().rope_kv_write(want, inv_freq, rot, 1.0, tok_pos, tok_seq, table, k1, v1, nh, nkv, hd, page, True)
    for bias in (b, None):
        if bias is None:
            want = K().gemm_pair(x, w, None)
            k1, v1 = junk_k.clone(), junk_v.clone()
            K().rope_kv_write(want, inv_freq, rot, 1.0, tok_pos, tok_seq, table, k1, v1, nh, nkv, hd, page, True)
        k2, v2 = junk_k.clone(), junk_v.clone()
        got = K().gemm_pair_rope(x, w, bias, None, tok_pos, tok_seq, table, inv_freq, rot, 1.0, nh, nkv, hd, page,
                                 k2, v2, True)
        close(got[:, :nh * hd], want[:, :nh * hd].double(), 1e-2, "rotated queries")
        close(k2, k1.double(), 1e-2, "key cache")
        assert torch.equal(v2, v1)                       # values are copied, not computed with
        # where no token lives, the pools are as they were
        touched = torch.zeros(n_pages, page, dtype=torch.bool)
        pages_of = table.cpu()
        for p_, s_ in zip(tok_pos.tolist(), tok_seq.tolist()):
            touched[pages_of[s_, p_ // page], p_ % page] = True
        free = ~touched.to(DEV)
        assert torch.equal(k2.permute(0, 2, 1, 3)[free], junk_k.permute(0, 2, 1, 3)[free])
        assert torch.equal(v2.permute(0, 2, 1, 3)[free], junk_v.permute(0, 2, 1, 3)[free])
        # without the cache write: the queries only
        k3, v3 = junk_k.clone(), junk_v.clone()
        got = K().gemm_pair_rope(x, w, bias, None, tok_pos, tok_seq, None, inv_freq, rot, 1.0, nh, nkv, hd, page,
                                 None, None, False)
        close(got[:, :nh * hd], want[:, :nh * hd].double(), 1e-2, "rotated queries, no cache write")
    torch.cuda.synchronize()
    assert K().gemm_pair_status() == 0


def test_gemm_pair_refuses_what_it_cannot_do():
    from exl3_server_b200.ops.lib import KernelLibraryError
    x = torch.zeros(300, 64, device=DEV).bfloat16()
    w = torch.zeros(24, 64, device=DEV).bfloat16()
    with pytest.raises(KernelLibraryError, match="multiples of 8"):
        K().gemm_pair(x[:, :60].contiguous(), w[:, :60].contiguous(), None)
    with pytest.raises(KernelLibraryError, match="multiples of 8"):
        K().gemm_pair(x, w[:20].contiguous(), None)
    with pytest.raises(KernelLibraryError, match="N of 16 with the gated"):
        K().gemm_pair(x, w, None, gated=True)
    with pytest.raises(KernelLibraryError, match="output is bfloat16"):
        K().gemm_pair(x, w, None, torch.float32)
    h = torch.zeros(300, 24, device=DEV)
    with pytest.raises(KernelLibraryError, match="scale that is not zero"):
        K().gemm_pair(x, w, None, resid=(h, 0.0, torch.ones(24, device=DEV)))


def test_gemm_skinny_refuses_what_it_cannot_do():
    from exl3_server_b200.ops.lib import KernelLibraryError
    x = torch.zeros(129, 64, device=DEV).bfloat16()
    w = torch.zeros(8, 64, device=DEV).bfloat16()
    with pytest.raises(KernelLibraryError, match="M <= 128"):
        K().gemm_skinny(x, w, None, torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="multiple of 8"):
        K().gemm_skinny(x[:20, :60].contiguous(), w[:, :60].contiguous(), None, torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="multiple of 16 when gated"):
        K().gemm_skinny(x[:20].contiguous(), w, None, torch.bfloat16, gated=True)


def test_gemv_refuses_what_it_cannot_do():
    from exl3_server_b200.ops.lib import KernelLibraryError
    x = torch.zeros(17, 64, device=DEV).bfloat16()
    w = torch.zeros(8, 64, device=DEV).bfloat16()
    with pytest.raises(KernelLibraryError, match="M <= 16"):
        K().gemv_bf16(x, w, None, torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="multiple of 8"):
        K().gemv_bf16(x[:2, :60].contiguous(), w[:, :60].contiguous(), None, torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="not on a CUDA device"):
        K().gemv_bf16(x.cpu(), w, None, torch.bfloat16)


# -- attention ---------------------------------------------------------------

class PagedCase:
    """Sequences with random keys and values scattered over shuffled pages."""

    def __init__(self, lens, new, nh, nkv, hd, dtype, seed=0, page=64, spare_pages=5):
        g = torch.Generator().manual_seed(seed)
        self.lens, self.new, self.nh, self.nkv, self.hd, self.page = lens, new, nh, nkv, hd, page
        B = len(lens)
        need = [(n + page - 1) // page for n in lens]
        n_pages = sum(need) + spare_pages
        perm = torch.randperm(n_pages, generator=g).tolist()
        width = max(need)
        table = torch.full((B, width), -1, dtype=torch.int32)
        self.k = [torch.randn(n, nkv, hd, generator=g).to(dtype) for n in lens]
        self.v = [torch.randn(n, nkv, hd, generator=g).to(dtype) for n in lens]
        kp = torch.randn(n_pages, nkv, page, hd, generator=g).to(dtype)      # stale junk in unused places
        vp = torch.randn(n_pages, nkv, page, hd, generator=g).to(dtype)
        it = iter(perm)
        for b in range(B):
            for i in range(need[b]):
                pg = next(it)
                table[b, i] = pg
                a, e = i * page, min(lens[b], (i + 1) * page)
                kp[pg, :, :e - a] = self.k[b][a:e].transpose(0, 1)
                vp[pg, :, :e - a] = self.v[b][a:e].transpose(0, 1)
        self.k_pool, self.v_pool, self.table = kp.to(DEV), vp.to(DEV), table.to(DEV)
        T = sum(new)
        self.q = torch.randn(T, nh, hd, generator=g).to(dtype)
        self.tok_seq = torch.tensor([b for b in range(B) for _ in range(new[b])], dtype=torch.int32, device=DEV)
        self.tok_pos = torch.tensor([lens[b] - new[b] + i for b in range(B) for i in range(new[b])],
                                    dtype=torch.int32, device=DEV)
        starts = [0]
        for n in new:
            starts.append(starts[-1] + n)
        self.row_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        self.row_pos0 = torch.tensor([lens[b] - new[b] for b in range(B)], dtype=torch.int32, device=DEV)

    def tiles(self, size):
        # any order is right; the engine lists the tiles with the most keys first
        B = len(self.new)
        order = sorted(((self.lens[b] - self.new[b] + a, b, a) for b in range(B) for a in range(0, self.new[b], size)),
                       reverse=True)
        seq = torch.tensor([b for _, b, _ in order], dtype=torch.int32, device=DEV)
        q0 = torch.tensor([a for _, _, a in order], dtype=torch.int32, device=DEV)
        return seq, q0

    def reference(self, window, scale):
        outs = []
        t = 0
        G = self.nh // self.nkv
        for b, (n, m) in enumerate(zip(self.lens, self.new)):
            k = self.k[b].double().repeat_interleave(G, dim=1)       # [n, nh, hd]
            v = self.v[b].double().repeat_interleave(G, dim=1)
            q = self.q[t:t + m].double()
            s = torch.einsum("qhd,khd->hqk", q, k) * scale
            qpos = torch.arange(n - m, n)[:, None]
            kpos = torch.arange(n)[None, :]
            allow = kpos <= qpos
            if window > 0:
                allow &= kpos > qpos - window
            s = s.masked_fill(~allow, float("-inf"))
            outs.append(torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v))
            t += m
        return torch.cat(outs).reshape(-1, self.nh * self.hd)


ATT_SHAPES = [  # heads, kv heads, head_dim
    (4, 2, 16), (4, 1, 32), (6, 3, 48), (3, 3, 64), (8, 2, 128), (5, 1, 80), (2, 2, 256),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 100])
def test_attn_tokens(dtype, nh, nkv, hd, window):
    # whole prompts and single tokens in one call, chunks of 128 keys so that several are merged
    case = PagedCase(lens=[300, 64, 1, 700], new=[300, 1, 1, 40], nh=nh, nkv=nkv, hd=hd, dtype=dtype, seed=hd + nh)
    T = case.q.shape[0]
    q = case.q.reshape(T, nh * hd).to(DEV).contiguous()
    out = torch.empty_like(q)
    scale = 0.7 / math.sqrt(hd)
    split = 128
    n = (max(case.lens) + split - 1) // split
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(T, nh, hd, n) // 4, device=DEV)
    K().attn_tokens(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                    nh, nkv, hd, 64, window, scale, split, n, scratch)
    close(out, case.reference(window, scale), 2e-6 if dtype == torch.float32 else 1e-2, "attn_tokens")


def test_attn_tokens_finds_one_far_key_among_many():
    """One key far back matches the query strongly: the output must be that
    key's value, not an average, and a window that excludes it must lose it."""
    nh = nkv = 2
    hd = 64
    case = PagedCase(lens=[900], new=[1], nh=nh, nkv=nkv, hd=hd, dtype=torch.float32, seed=3)
    far = 37
    kp, table = case.k_pool, case.table
    pg = int(table[0, far // 64])
    qv = case.q[0].clone()                                                    # [nh, hd]
    kp[pg, :, far % 64] = (qv * 40.0 / qv.norm(dim=-1, keepdim=True)).to(DEV)  # score stands out by far
    case.k[0][far] = kp[pg, :, far % 64].cpu()
    q = (case.q.reshape(1, nh * hd) * 1.0).to(DEV).contiguous()
    out = torch.empty_like(q)
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(1, nh, hd, 4) // 4, device=DEV)
    K().attn_tokens(q, q.stride(0), out, kp, case.v_pool, table, case.tok_pos, case.tok_seq, 1, nh, nkv, hd, 64, 0,
                    1.0, 256, 4, scratch)
    close(out, case.v[0][far].reshape(1, -1), 1e-3, "far key")
    close(out, case.reference(0, 1.0), 2e-6, "far key vs reference")
    K().attn_tokens(q, q.stride(0), out, kp, case.v_pool, table, case.tok_pos, case.tok_seq, 1, nh, nkv, hd, 64, 800,
                    1.0, 256, 4, scratch)
    close(out, case.reference(800, 1.0), 2e-6, "window excludes the far key")
    assert float((out.cpu() - case.v[0][far].reshape(1, -1)).abs().max()) > 0.1


@pytest.mark.parametrize("nh,nkv,hd", [(3, 3, 64), (4, 2, 64), (8, 1, 64), (16, 2, 64), (5, 5, 64), (6, 2, 64),
                                       (5, 1, 64), (3, 3, 128), (8, 1, 128), (8, 2, 128), (6, 1, 128), (9, 3, 128),
                                       # 9 to 16 query heads per kv head: two blocks of instruction columns
                                       (16, 1, 64), (9, 1, 64), (26, 2, 64), (32, 2, 128), (12, 1, 128), (30, 3, 128)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("split", [64, 256])
def test_attn_decode(nh, nkv, hd, window, split):
    # single tokens and short prompts in one call, positions at both sides of page and chunk edges
    lens = [300, 64, 1, 700, 65, 256, 257, 128, 513]
    new = [1, 1, 1, 3, 1, 1, 1, 2, 1]
    case = PagedCase(lens=lens, new=new, nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=nh + split)
    T = case.q.shape[0]
    q = case.q.reshape(T, nh * hd).to(DEV).contiguous()
    out = torch.empty_like(q)
    scale = 0.7 / math.sqrt(hd)
    n = (max(lens) + split - 1) // split
    if window > 0:
        n = min(n, (window + split - 2) // split + 1)
    assert K().attn_decode_supported(torch.bfloat16, T, nh, nkv, hd, 64, split, n)
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(T, nh, hd, n) // 4, device=DEV)
    for _ in range(2):                                  # the second call finds the counters as the first left them
        out.fill_(7.0)
        K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                        nh, nkv, hd, 64, window, scale, split, n, scratch)
        close(out, case.reference(window, scale), 1e-2, "attn_decode")
    for parts in (2, 4, 8, 16):
        if (nh // nkv) % parts == 0:
            # the query heads of a kv head as several groups of work: the same numbers
            halves = torch.full_like(out, 7.0)
            K().attn_decode(q, q.stride(0), halves, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq,
                            T, nh, nkv, hd, 64, window, scale, split, n, scratch, head_split=parts)
            assert torch.equal(halves, out), parts
    assert K().attn_decode_status() == 0


@pytest.mark.parametrize("nh,nkv,hd", [(4, 4, 64), (16, 2, 64), (32, 2, 128), (12, 4, 128), (9, 1, 64), (36, 36, 64)])
@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("split", [256, 1024])
def test_attn_decode_merges_in_the_block(nh, nkv, hd, window, split):
    """A block per (token, group of heads) whose warps take the item's chunks and merge them in shared memory:
    sequences with one to four chunks (and a token whose window ends inside a chunk), with and without the query
    heads of a kv head cut into groups, against the reference and against the merge through global memory."""
    lens = [1000, 64, 1, 700, 257, 256, 513, 1024, 769]
    new = [1, 1, 1, 2, 1, 1, 1, 1, 1]
    case = PagedCase(lens=lens, new=new, nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=nh + split)
    T = case.q.shape[0]
    q = case.q.reshape(T, nh * hd).to(DEV).contiguous()
    scale = 0.7 / math.sqrt(hd)
    n = (max(lens) + split - 1) // split
    if window > 0:
        n = min(n, (window + split - 2) // split + 1)
    assert n <= 4
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(T, nh, hd, n) // 4, device=DEV)
    want = case.reference(window, scale)
    through_memory = torch.full_like(q, 7.0)
    K().attn_decode(q, q.stride(0), through_memory, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                    nh, nkv, hd, 64, window, scale, split, n, scratch)
    for parts in (1, 2, 4):
        if (nh // nkv) % parts:
            continue
        for _ in range(2):
            out = torch.full_like(q, 7.0)
            K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                            nh, nkv, hd, 64, window, scale, split, n, None, head_split=parts, in_block=True)
            close(out, want, 1e-2, f"attn_decode, merged in the block, {parts} groups per kv head")
            close(out, through_memory.double(), 1e-2, "the two ways of merging")
    assert K().attn_decode_status() == 0
    from exl3_server_b200.ops.lib import KernelLibraryError
    with pytest.raises(KernelLibraryError, match="up to 4 chunks"):
        K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                        nh, nkv, hd, 64, 0, scale, 64, 16, None, in_block=True)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 4, 64), (16, 2, 64), (32, 2, 128), (12, 4, 128), (36, 36, 64)])
@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("split", [128, 256])
def test_attn_decode_merges_in_a_cluster_of_two_blocks(nh, nkv, hd, window, split):
    """A cluster of two blocks per (token, group of heads): eight warps take the item's up to eight chunks, and the
    first block merges them, reading the second one's records out of its shared memory.  Sequences with one to eight
    chunks (the ones with at most four leave the second block nothing to do), against the reference and against
    the merge through global memory."""
    lens = [1000, 64, 1, 700, 257, 256, 513, 1024, 769, 2 * split + 1, 6 * split]
    lens = [min(n, 8 * split) for n in lens]
    new = [1, 1, 1, 2, 1, 1, 1, 1, 1, 1, 1]
    case = PagedCase(lens=lens, new=new, nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=nh + split + 1)
    T = case.q.shape[0]
    q = case.q.reshape(T, nh * hd).to(DEV).contiguous()
    scale = 0.7 / math.sqrt(hd)
    n = (max(lens) + split - 1) // split
    if window > 0:
        n = min(n, (window + split - 2) // split + 1)
    assert n <= 8
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(T, nh, hd, n) // 4, device=DEV)
    want = case.reference(window, scale)
    through_memory = torch.full_like(q, 7.0)
    K().attn_decode(q, q.stride(0), through_memory, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                    nh, nkv, hd, 64, window, scale, split, n, scratch)
    for parts in (1, 2, 4):
        if (nh // nkv) % parts:
            continue
        for _ in range(2):
            out = torch.full_like(q, 7.0)
            K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                            nh, nkv, hd, 64, window, scale, split, n, None, head_split=parts, in_block=2)
            close(out, want, 1e-2, f"attn_decode, merged in a cluster, {parts} groups per kv head")
            close(out, through_memory.double(), 1e-2, "the two ways of merging")
    assert K().attn_decode_status() == 0
    from exl3_server_b200.ops.lib import KernelLibraryError
    with pytest.raises(KernelLibraryError, match="up to 8"):
        K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                        nh, nkv, hd, 64, 0, scale, 64, 16, None, in_block=2)


@pytest.mark.parametrize("nh,nkv,hd", [(16, 2, 64), (32, 2, 128), (12, 2, 128), (8, 1, 64), (4, 2, 64), (16, 1, 128)])
@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("in_block", [1, 2])
def test_attn_decode_with_two_groups_of_heads_walking_the_same_pages(nh, nkv, hd, window, in_block):
    """Two groups of query heads of a kv head in one block, their warps reading the same rings of pages: the very
    numbers that a block per group gives, and the reference's."""
    split = 128
    lens = [1000, 64, 1, 700, 257, 256, 513, 1024, 769, 2 * split + 1, 6 * split]
    lens = [min(n, 4 * in_block * split) for n in lens]
    case = PagedCase(lens=lens, new=[1, 1, 1, 2, 1, 1, 1, 1, 1, 1, 1], nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16,
                     seed=nh + hd + in_block)
    T = case.q.shape[0]
    q = case.q.reshape(T, nh * hd).to(DEV).contiguous()
    scale = 0.7 / math.sqrt(hd)
    n = (max(lens) + split - 1) // split
    if window > 0:
        n = min(n, (window + split - 2) // split + 1)
    want = case.reference(window, scale)
    group = nh // nkv
    ran = 0
    for parts in (2, 4, 8, 16):
        if group % parts or group // parts > 8:
            continue
        outs = []
        for twins in (1, 2, 2):
            out = torch.full_like(q, 7.0)
            K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                            nh, nkv, hd, 64, window, scale, split, n, None, head_split=parts, in_block=in_block,
                            twins=twins)
            close(out, want, 1e-2, f"{parts} groups per kv head, twins {twins}")
            outs.append(out)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
        ran += 1
    assert ran and K().attn_decode_status() == 0
    from exl3_server_b200.ops.lib import KernelLibraryError
    with pytest.raises(KernelLibraryError, match="twins is 1 or 2"):
        K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                        nh, nkv, hd, 64, window, scale, split, n, None, head_split=1, in_block=in_block, twins=2)
    with pytest.raises(KernelLibraryError, match="twins is 1 or 2"):
        scratch = torch.zeros(K().attn_tokens_scratch_bytes(T, nh, hd, n) // 4, device=DEV)
        K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                        nh, nkv, hd, 64, window, scale, split, n, scratch, head_split=2, in_block=0, twins=2)


@pytest.mark.parametrize("hd", [64, 128])
def test_attn_decode_many_items_per_warp(hd):
    # more work items than the grid has warps: every warp's ring of pages runs across the ends of items,
    # among them empty chunks of the shorter sequences
    nh, nkv = 8, 4
    g = torch.Generator().manual_seed(5)
    lens = [int(x) for x in torch.randint(1, 1500, (48,), generator=g)]
    case = PagedCase(lens=lens, new=[1] * len(lens), nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=11)
    T = case.q.shape[0]
    q = case.q.reshape(T, nh * hd).to(DEV).contiguous()
    out = torch.empty_like(q)
    split = 256
    n = (max(lens) + split - 1) // split
    assert T * nkv * n > 148 * 4
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(T, nh, hd, n) // 4, device=DEV)
    K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                    nh, nkv, hd, 64, 0, 0.125, split, n, scratch)
    close(out, case.reference(0, 0.125), 1e-2, "attn_decode, many items")
    # one chunk for everything: no merge, results written directly
    n1 = 1
    K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                    nh, nkv, hd, 64, 0, 0.125, 2048, n1, None)
    close(out, case.reference(0, 0.125), 1e-2, "attn_decode, one chunk")
    assert K().attn_decode_status() == 0


@pytest.mark.parametrize("nh,nkv,hd", [(8, 1, 64), (14, 2, 128), (4, 1, 128), (16, 1, 128), (22, 2, 64)])
def test_attn_decode_merges_many_chunks_of_grouped_heads(nh, nkv, hd):
    # so many chunks for each token that the heads of a group are merged in several passes
    lens = [2100, 1, 2049, 640]
    case = PagedCase(lens=lens, new=[1] * len(lens), nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=21)
    T = case.q.shape[0]
    q = case.q.reshape(T, nh * hd).to(DEV).contiguous()
    out = torch.empty_like(q)
    split = 64
    n = (max(lens) + split - 1) // split
    assert (nh // nkv) * n > 256 or nh // nkv < 8
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(T, nh, hd, n) // 4, device=DEV)
    for _ in range(2):
        out.fill_(7.0)
        K().attn_decode(q, q.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, T,
                        nh, nkv, hd, 64, 0, 0.125, split, n, scratch)
        close(out, case.reference(0, 0.125), 1e-2, "attn_decode, many chunks of grouped heads")
    assert K().attn_decode_status() == 0


def test_attn_decode_finds_one_far_key_among_many():
    nh = nkv = 2
    hd = 64
    case = PagedCase(lens=[900], new=[1], nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=3)
    far = 37
    kp, table = case.k_pool, case.table
    pg = int(table[0, far // 64])
    qv = case.q[0].float()
    kp[pg, :, far % 64] = (qv * 40.0 / qv.norm(dim=-1, keepdim=True)).to(torch.bfloat16).to(DEV)
    case.k[0][far] = kp[pg, :, far % 64].cpu()
    q = case.q.reshape(1, nh * hd).to(DEV).contiguous()
    out = torch.empty_like(q)
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(1, nh, hd, 4) // 4, device=DEV)
    K().attn_decode(q, q.stride(0), out, kp, case.v_pool, table, case.tok_pos, case.tok_seq, 1, nh, nkv, hd, 64, 0,
                    1.0, 256, 4, scratch)
    close(out, case.v[0][far].reshape(1, -1), 1e-2, "far key")
    close(out, case.reference(0, 1.0), 1e-2, "far key vs reference")
    K().attn_decode(q, q.stride(0), out, kp, case.v_pool, table, case.tok_pos, case.tok_seq, 1, nh, nkv, hd, 64, 800,
                    1.0, 256, 4, scratch)
    close(out, case.reference(800, 1.0), 1e-2, "window excludes the far key")
    assert float((out.cpu().float() - case.v[0][far].reshape(1, -1).float()).abs().max()) > 0.1


@pytest.mark.parametrize("nh,nkv,hd", [(3, 3, 64), (8, 1, 64), (16, 2, 64), (4, 2, 128), (8, 1, 128), (16, 1, 64),
                                       (32, 2, 128), (10, 1, 128)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("rotary", [True, False])
@pytest.mark.parametrize("split", [64, 256, 2048])
def test_attn_decode_rotates_and_writes_the_new_token(nh, nkv, hd, window, rotary, split):
    """The kernel takes each token's own key and value from the projection's output: the cache holds junk at
    the token's place before the call and the rotated key and the value after it."""
    rot = hd if rotary else 0
    lens = [300, 64, 1, 700, 65, 256, 257, 128, 513, 2]         # last positions at both sides of page and chunk edges
    B = len(lens)
    case = PagedCase(lens=lens, new=[1] * B, nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=nh + split + rot)
    g = torch.Generator().manual_seed(99)
    q_raw = torch.randn(B, nh, hd, generator=g).to(torch.bfloat16)
    k_raw = torch.randn(B, nkv, hd, generator=g).to(torch.bfloat16)
    v_raw = torch.randn(B, nkv, hd, generator=g).to(torch.bfloat16)
    theta, pos_scale = 10000.0, 1.0
    inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64),
                         -2.0 * torch.arange(0, hd // 2, dtype=torch.float64) / hd).to(torch.float32)

    def rotated(x, pos):                                        # [heads, hd] at one position
        if not rot:
            return x
        a = (torch.tensor(float(pos), dtype=torch.float32) * pos_scale * inv_freq).double()
        x0, x1 = x[:, :hd // 2].double(), x[:, hd // 2:].double()
        return torch.cat([x0 * a.cos() - x1 * a.sin(), x1 * a.cos() + x0 * a.sin()], dim=1).to(torch.bfloat16)

    for b in range(B):
        pos = lens[b] - 1
        case.q[b] = rotated(q_raw[b], pos)
        case.k[b][pos] = rotated(k_raw[b], pos)
        case.v[b][pos] = v_raw[b]
        pg = int(case.table[b, pos // 64])
        case.k_pool[pg, :, pos % 64] = 100.0                   # not written yet: must not be read as a key
        case.v_pool[pg, :, pos % 64] = -100.0
    qkv = torch.cat([q_raw.reshape(B, -1), k_raw.reshape(B, -1), v_raw.reshape(B, -1)], dim=1).to(DEV).contiguous()
    out = torch.empty((B, nh * hd), dtype=torch.bfloat16, device=DEV)
    head_split = 2 if (nh // nkv) % 2 == 0 and split == 256 else 1     # two groups of work per kv head in some cases
    scale = 0.7 / math.sqrt(hd)
    n = (max(lens) + split - 1) // split
    if window > 0:
        n = min(n, (window + split - 2) // split + 1)
    scratch = torch.zeros(K().attn_tokens_scratch_bytes(B, nh, hd, n) // 4, device=DEV)
    K().attn_decode(qkv, qkv.stride(0), out, case.k_pool, case.v_pool, case.table, case.tok_pos, case.tok_seq, B,
                    nh, nkv, hd, 64, window, scale, split, n, scratch,
                    inv_freq=(K().rotary_table(inv_freq) if split == 256 else inv_freq).to(DEV), rot=rot,
                    pos_scale=pos_scale, write_new=True, head_split=head_split)
    close(out, case.reference(window, scale), 1e-2, "attn_decode, own key and value")

    def written():
        for b in range(B):
            pos = lens[b] - 1
            pg = int(case.table[b, pos // 64])
            close(case.k_pool[pg, :, pos % 64], case.k[b][pos], 1e-2, "key written to the cache")
            assert torch.equal(case.v_pool[pg, :, pos % 64].cpu(), v_raw[b])
    written()
    # the same with a block, and a cluster of two, per item; and with two groups of heads of a kv head per block
    group = nh // nkv
    for in_block in (1, 2):
        if n > 4 * in_block:
            continue
        for twins in (1, 2):
            parts = 2 if group % 2 == 0 else 1
            if twins == 2 and (parts != 2 or group // parts > 8):
                continue
            for b in range(B):
                pos = lens[b] - 1
                pg = int(case.table[b, pos // 64])
                case.k_pool[pg, :, pos % 64] = 100.0
                case.v_pool[pg, :, pos % 64] = -100.0
            other = torch.empty_like(out)
            K().attn_decode(qkv, qkv.stride(0), other, case.k_pool, case.v_pool, case.table, case.tok_pos,
                            case.tok_seq, B, nh, nkv, hd, 64, window, scale, split, n, None,
                            inv_freq=inv_freq.to(DEV), rot=rot, pos_scale=pos_scale, write_new=True,
                            head_split=parts, in_block=in_block, twins=twins)
            close(other, case.reference(window, scale), 1e-2, f"in_block {in_block}, twins {twins}")
            written()
    assert K().attn_decode_status() == 0


def test_attn_decode_is_refused_for_other_shapes():
    assert K().attn_decode_supported(torch.bfloat16, 8, 4, 4, 64, 64, 256, 16)
    assert not K().attn_decode_supported(torch.float32, 8, 4, 4, 64, 64, 256, 16)
    assert K().attn_decode_supported(torch.bfloat16, 8, 4, 4, 128, 64, 256, 16)
    assert not K().attn_decode_supported(torch.bfloat16, 8, 4, 4, 96, 64, 256, 16)
    assert K().attn_decode_supported(torch.bfloat16, 8, 16, 1, 64, 64, 256, 16)          # 16 query heads per kv head
    assert not K().attn_decode_supported(torch.bfloat16, 8, 17, 1, 64, 64, 256, 16)
    assert not K().attn_decode_supported(torch.bfloat16, 8, 40, 2, 128, 64, 256, 16)
    assert not K().attn_decode_supported(torch.bfloat16, 8, 4, 4, 64, 64, 100, 16)
    assert not K().attn_decode_supported(torch.bfloat16, 5000, 4, 4, 64, 64, 256, 16)
    assert not K().attn_decode_supported(torch.bfloat16, 8, 4, 4, 64, 64, 256, 1000)


@pytest.mark.parametrize("nh,nkv,hd", [(3, 3, 64), (4, 2, 64), (8, 1, 64), (3, 3, 128), (8, 2, 128), (5, 1, 128)])
@pytest.mark.parametrize("window", [0, 24, 100])
def test_attn_prefill_tc(nh, nkv, hd, window):
    case = PagedCase(lens=[300, 64, 1, 700, 65, 128, 129], new=[300, 64, 1, 200, 65, 1, 129], nh=nh, nkv=nkv, hd=hd,
                     dtype=torch.bfloat16, seed=hd + nh + window)
    T = case.q.shape[0]
    buf = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    buf[:, :nh * hd] = case.q.reshape(T, nh * hd).to(DEV)
    out = torch.empty(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    scale = 1.3 / math.sqrt(hd)
    assert K().attn_prefill_tc_supported(torch.bfloat16, hd, 64)
    tile_seq, tile_q0 = case.tiles(128)
    K().attn_prefill_tc(buf, buf.stride(0), out, case.k_pool, case.v_pool, case.table, case.row_start, case.row_pos0,
                        tile_seq, tile_q0, tile_seq.numel(), nh, nkv, hd, 64, window, scale)
    torch.cuda.synchronize()
    assert K().attn_prefill_tc_status() == 0
    close(out, case.reference(window, scale), 1e-2, "attn_prefill_tc")
    # a tile a block, four blocks per SM with one S buffer (heads of 64), or two tiles a block (the list's first with
    # its last, and so on): the same arithmetic in the same order
    outs = []
    for variant in ((1, 2, 3) if hd == 64 else (1, 3)):
        o = torch.full_like(out, 3.0)
        K().attn_prefill_tc(buf, buf.stride(0), o, case.k_pool, case.v_pool, case.table, case.row_start,
                            case.row_pos0, tile_seq, tile_q0, tile_seq.numel(), nh, nkv, hd, 64, window, scale,
                            variant=variant)
        close(o, case.reference(window, scale), 1e-2, f"attn_prefill_tc variant {variant}")
        outs.append(o)
    for o in outs[1:]:
        assert torch.equal(outs[0], o)
    torch.cuda.synchronize()
    assert K().attn_prefill_tc_status() == 0


@pytest.mark.parametrize("hd", [64, 128])
def test_attn_prefill_tc_moves_its_reference_maximum(hd):
    """Keys grow page by page, so every row's running maximum rises by far more than the kernel lets its
    exponentials' reference lag behind: the accumulator in tensor memory is rescaled again and again."""
    nh, nkv = 2, 1
    case = PagedCase(lens=[700, 330], new=[700, 200], nh=nh, nkv=nkv, hd=hd, dtype=torch.bfloat16, seed=41)
    for b, n in enumerate(case.lens):
        for pos in range(n):
            f = 1.0 + 3.0 * (pos // 64)
            case.k[b][pos] = (case.k[b][pos].float() * f).to(torch.bfloat16)
            pg = int(case.table[b, pos // 64])
            case.k_pool[pg, :, pos % 64] = case.k[b][pos].to(DEV)
    T = case.q.shape[0]
    buf = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    buf[:, :nh * hd] = case.q.reshape(T, nh * hd).to(DEV)
    out = torch.empty(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    tile_seq, tile_q0 = case.tiles(128)
    for variant in ((1, 2, 3) if hd == 64 else (1, 3)):
        out.fill_(3.0)
        K().attn_prefill_tc(buf, buf.stride(0), out, case.k_pool, case.v_pool, case.table, case.row_start,
                            case.row_pos0, tile_seq, tile_q0, tile_seq.numel(), nh, nkv, hd, 64, 0, scale,
                            variant=variant)
        torch.cuda.synchronize()
        assert K().attn_prefill_tc_status() == 0
        close(out, case.reference(0, scale), 1e-2, f"attn_prefill_tc, rising maximum, variant {variant}")


def test_attn_prefill_is_refused_for_other_shapes():
    assert not K().attn_prefill_tc_supported(torch.float32, 64, 64)
    assert not K().attn_prefill_tc_supported(torch.bfloat16, 48, 64)
    assert not K().attn_prefill_tc_supported(torch.bfloat16, 64, 32)


# -- rotary + cache write ------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (6, 3, 48, 48), (2, 1, 64, 32), (3, 3, 80, 0),
                                           (2, 1, 32, 24), (36, 36, 64, 64)])
def test_rope_kv_write(dtype, nh, nkv, hd, rot):
    torch.manual_seed(6)
    page = 64
    lens_before, new = [70, 0, 130], [3, 5, 1]
    B = 3
    n_pages = 8
    table = torch.tensor([[5, 2, -1], [7, -1, -1], [0, 3, 6]], dtype=torch.int32, device=DEV)
    T = sum(new)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(dtype)
    orig = qkv.clone()
    tok_seq = torch.tensor([b for b in range(B) for _ in range(new[b])], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lens_before[b] + i for b in range(B) for i in range(new[b])], dtype=torch.int32, device=DEV)
    kp = torch.zeros(n_pages, nkv, page, hd, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    theta = 2500.0
    inv = (theta ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(1, rot))).float().to(DEV)
    K().rope_kv_write(qkv, inv, rot, 1.0, tok_pos, tok_seq, table, kp, vp, nh, nkv, hd, page, True)

    def rotate(x, pos):                                  # x [heads, hd] float64
        if rot == 0:
            return x
        a = pos * inv.double().cpu()
        c, s = torch.cos(a), torch.sin(a)
        x0, x1, rest = x[:, :rot // 2], x[:, rot // 2:rot], x[:, rot:]
        return torch.cat([x0 * c - x1 * s, x1 * c + x0 * s, rest], dim=-1)

    tol = 3e-6 if dtype == torch.float32 else 1e-2
    for t in range(T):
        b, pos = int(tok_seq[t]), int(tok_pos[t])
        row = orig[t].double().cpu()
        q = row[:nh * hd].reshape(nh, hd)
        k = row[nh * hd:(nh + nkv) * hd].reshape(nkv, hd)
        v = row[(nh + nkv) * hd:].reshape(nkv, hd)
        close(qkv[t, :nh * hd].reshape(nh, hd), rotate(q, pos), tol, "q")
        pg = int(table[b, pos // page])
        close(kp[pg, :, pos % page], rotate(k, pos), tol, "k in cache")
        assert torch.equal(vp[pg, :, pos % page].cpu().double(), v), "v in cache"
    written = sum(new) * nkv * hd
    assert int((vp != 0).sum()) <= written               # nothing else was touched


@pytest.mark.parametrize("hd", [64, 80])                        # the 16-byte kernel and the general one
def test_rope_angles_stay_exact_at_large_positions(hd):
    """At position 150,000 a frequency rounded to float32 puts the fastest pairs' angles off by up to 1e-2
    radians; with the table's second row (what the rounding lost) the kernel's float32 angles stay right."""
    nh, nkv = 2, 1
    pos = [150001, 99999, 31337]
    T = len(pos)
    g = torch.Generator().manual_seed(8)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g)
    f64 = torch.pow(torch.tensor(500000.0, dtype=torch.float64), -2.0 * torch.arange(0, hd // 2, dtype=torch.float64) / hd)
    ang = torch.tensor(pos, dtype=torch.float64)[:, None] * f64[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x = qkv.double().reshape(T, nh + 2 * nkv, hd)[:, :nh]
    x0, x1 = x[..., :hd // 2], x[..., hd // 2:]
    want = torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)
    tok_pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    errs = []
    for tab in (K().rotary_table(f64).to(DEV), f64.float().to(DEV)):
        buf = qkv.to(DEV).clone()
        K().rope_kv_write(buf, tab, hd, 1.0, tok_pos, tok_seq, table, None, None, nh, nkv, hd, 64, False)
        got = buf.cpu().double().reshape(T, nh + 2 * nkv, hd)[:, :nh]
        errs.append(float((got - want).abs().max()))
    assert errs[0] < 3e-6, errs          # float32 sine and cosine of an angle that is right
    assert errs[1] > 1e-4, errs          # the plain table shows what the second row is for


# -- sampling ------------------------------------------------------------------

@pytest.mark.parametrize("V", [7, 1000, 122753])
def test_argmax_first_maximum(V):
    torch.manual_seed(7)
    x = torch.randn(5, V, device=DEV)
    x[1, V // 2] = 50.0
    x[1, V - 1] = 50.0                                   # a tie: the first wins
    x[2, 0] = 60.0
    x[3, V - 1] = 70.0
    got = K().argmax(x).cpu().tolist()
    assert got == [int(torch.argmax(x[0])), V // 2, 0, V - 1, int(torch.argmax(x[4]))]


class _FixedU:
    """A generator that hands out one given number."""
    def __init__(self, u):
        self.u = u

    def uniform01(self):
        return self.u


def _host_ranking(logits, opt):
    """The host sampler's candidates in its order, and the running sums of their probabilities (float64)."""
    x = logits.astype(np.float32)
    m = min(x.shape[0], 2048)
    idx = np.argsort(-x, kind="stable")[:m]
    inv_t = np.float32(1.0) / np.float32(opt.temperature)
    probs = np.exp(x[idx] * inv_t - x[idx[0]] * inv_t).astype(np.float32)
    return idx, np.cumsum(probs.astype(np.float64))


@pytest.mark.parametrize("V", [300, 5000, 122753])
def test_sample_filtered_agrees_with_the_host_sampler(V):
    from exl3_server_b200.sampling import SampleOptions
    from exl3_server_b200.sampling.host import sample_token
    rng = np.random.default_rng(V)
    option_sets = [SampleOptions(temperature=0.7), SampleOptions(temperature=1.3, top_k=5),
                   SampleOptions(temperature=1.0, top_p=0.9), SampleOptions(temperature=2.0, top_p=0.5, top_k=50),
                   SampleOptions(temperature=1.0, min_p=0.05),
                   SampleOptions(temperature=0.9, min_p=0.02, top_p=0.8, top_k=40),
                   SampleOptions(temperature=0.0), SampleOptions(temperature=30.0)]
    R = len(option_sets)
    logits = (3.0 * rng.normal(size=(R, V))).astype(np.float32)
    dev_logits = torch.from_numpy(logits).to(DEV)
    near = 0
    for u in [0.0, 1e-9, 0.013, 0.25, 0.5, 0.77, 0.93, 0.999999] + rng.random(24).tolist():
        rows = torch.tensor([[o.temperature, o.top_k, o.top_p, o.min_p, u] for o in option_sets], dtype=torch.float64)
        got = K().sample_filtered(dev_logits, rows.to(DEV)).cpu().tolist()
        for r, o in enumerate(option_sets):
            want = sample_token(logits[r], o, [], _FixedU(u))
            if got[r] == want:
                continue
            # float32 exponentials may differ in their last bit between host and device: the two may part only
            # where u falls on the border between two neighbours of the ranking
            idx, acc = _host_ranking(logits[r], o)
            i, j = int(np.nonzero(idx == want)[0][0]), int(np.nonzero(idx == got[r])[0][0])
            assert abs(i - j) == 1, (V, u, r, want, got[r])
            near += 1
    assert near <= 2, near


def test_sample_filtered_ranks_equal_logits_by_index():
    """Many tokens share each value (logits rounded to halves), also across the 2048th place: the ranking takes
    the smaller index first, as the host's stable sort does."""
    from exl3_server_b200.sampling import SampleOptions
    from exl3_server_b200.sampling.host import sample_token
    rng = np.random.default_rng(5)
    V = 9000
    logits = (np.round(2.0 * rng.normal(size=(3, V))) / 2.0).astype(np.float32)
    logits[2, :] = 1.0                                   # one value only: the first 2048 indices are the candidates
    dev_logits = torch.from_numpy(logits).to(DEV)
    opts = [SampleOptions(temperature=1.0), SampleOptions(temperature=5.0, top_k=700), SampleOptions(temperature=1.0)]
    for u in [0.0, 0.2, 0.41, 0.63, 0.87, 0.99]:
        rows = torch.tensor([[o.temperature, o.top_k, o.top_p, o.min_p, u] for o in opts], dtype=torch.float64)
        got = K().sample_filtered(dev_logits, rows.to(DEV)).cpu().tolist()
        want = [sample_token(logits[r], o, [], _FixedU(u)) for r, o in enumerate(opts)]
        assert got == want, (u, got, want)
        assert want[2] < 2048


def test_sample_filtered_keeps_to_the_2048_most_probable():
    rng = np.random.default_rng(0)
    V = 5000
    logits = rng.normal(size=(1, V)).astype(np.float32)
    allowed = set(np.argsort(-logits[0])[:2048].tolist())
    dev_logits = torch.from_numpy(logits).to(DEV).repeat(512, 1).contiguous()
    rows = torch.tensor([[50.0, 0, 1.0, 0.0, u] for u in rng.random(512)], dtype=torch.float64)
    picks = set(K().sample_filtered(dev_logits, rows.to(DEV)).cpu().tolist())
    assert picks <= allowed and len(picks) > 400


def test_sample_filtered_distribution():
    x = torch.log(torch.tensor([[0.6, 0.3, 0.1]], device=DEV)).repeat(4096, 1).contiguous()
    u = torch.rand(4096, dtype=torch.float64)
    one, zero = torch.ones(4096, dtype=torch.float64), torch.zeros(4096, dtype=torch.float64)
    rows = torch.stack([one, zero, one, zero, u], dim=1).contiguous()
    got = K().sample_filtered(x, rows.to(DEV))
    freq = torch.bincount(got.long(), minlength=3).double().cpu() / 4096
    assert torch.allclose(freq, torch.tensor([0.6, 0.3, 0.1], dtype=torch.float64), atol=0.03)


def test_sample_penalties_as_on_the_host():
    from exl3_server_b200.sampling import SampleOptions, apply_penalties
    rng = np.random.default_rng(9)
    V, R = 1000, 3
    logits = (2.0 * rng.normal(size=(R, V))).astype(np.float32)
    opts = [SampleOptions(repetition_penalty=1.3, presence_penalty=0.4, frequency_penalty=0.15),
            SampleOptions(), SampleOptions(repetition_penalty=0.8, frequency_penalty=0.3)]
    contexts = [rng.integers(0, V, size=n).tolist() for n in (400, 50, 7)]
    want = logits.copy()
    counts = []
    for r in range(R):
        apply_penalties(want[r], opts[r], contexts[r])
        counts.append(torch.bincount(torch.tensor(contexts[r]), minlength=V).to(torch.int32).to(DEV))
    ptrs = torch.tensor([c.data_ptr() if o.has_penalties else 0 for c, o in zip(counts, opts)], dtype=torch.int64).to(DEV)
    params = torch.tensor([[o.repetition_penalty, o.presence_penalty, o.frequency_penalty] for o in opts])
    dev = torch.from_numpy(logits).to(DEV)
    K().sample_penalties(dev, ptrs, params.to(DEV))
    assert np.array_equal(dev.cpu().numpy(), want)
    # the chosen tokens join the counts of the rows that keep counts
    ids = torch.tensor([5, 6, 7], dtype=torch.int32, device=DEV)
    before = [int(c[t]) for c, t in zip(counts, (5, 6, 7))]
    K().sample_count(ptrs, ids, V)
    after = [int(c[t]) for c, t in zip(counts, (5, 6, 7))]
    assert after == [before[0] + 1, before[1], before[2] + 1]
