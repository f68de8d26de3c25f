"""Python faces of the CUDA entry points.

Every function takes torch tensors that live on the current CUDA device,
launches on torch's current stream and raises ``KernelLibraryError`` when the
entry point refuses its arguments.  There is no other implementation behind
these names: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .lib import KernelLibraryError, library

DT_F32, DT_BF16 = 0, 1

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_void_p = ctypes.c_void_p
_c_size_t = ctypes.c_size_t
_c_int64 = ctypes.c_int64


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return DT_F32
    if dt == torch.bfloat16:
        return DT_BF16
    raise KernelLibraryError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    if not t.is_cuda:
        raise KernelLibraryError("kernel called with a tensor that is not on a CUDA device; "
                                 "there is no CPU implementation of the product path")
    return _c_void_p(t.data_ptr())


def _stream() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        msg = library().exl3_last_error().decode("utf-8", "replace")
        raise KernelLibraryError(f"{what} failed (code {rc}): {msg}")


def launch_count() -> int:
    """Kernel launches made through the library so far."""
    lib = library()
    lib.exl3_launch_count.restype = ctypes.c_longlong
    return int(lib.exl3_launch_count())


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelLibraryError(f"{name} must be contiguous")


# ---------------------------------------------------------------------------

def embed(ids: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]] * scale`` as float32 rows."""
    T = ids.numel()
    V, H = table.shape
    _contig(table, "table")
    if ids.dtype != torch.int32:
        raise KernelLibraryError("embed: ids must be int32")
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(library().exl3_embed(_ptr(ids), _ptr(table), _c_int(dtype_code(table.dtype)), _ptr(out),
                                _c_int(T), _c_int(H), _c_int(V), _c_float(scale), _stream()), "embed")
    return out


def add_rmsnorm(h: torch.Tensor, y: Optional[torch.Tensor], y_scale: float, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, out_scale: float = 1.0, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += y * y_scale`` (when y is given), then RMSNorm of the rows of h
    (all, or those listed in ``rows``) times ``weight`` times ``out_scale``."""
    T, H = h.shape
    if h.dtype != torch.float32:
        raise KernelLibraryError("add_rmsnorm: the residual stream must be float32")
    _contig(h, "h")
    if y is not None:
        _contig(y, "y")
        if y.shape != h.shape:
            raise KernelLibraryError(f"add_rmsnorm: y is {tuple(y.shape)}, h is {tuple(h.shape)}")
    if weight.numel() != H:
        raise KernelLibraryError(f"add_rmsnorm: weight has {weight.numel()} elements, rows have {H}")
    n = T if rows is None else rows.numel()
    if rows is not None and rows.dtype != torch.int32:
        raise KernelLibraryError("add_rmsnorm: rows must be int32")
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=h.device)
    _check(library().exl3_add_rmsnorm(
        _ptr(h), _ptr(y), _c_int(dtype_code(y.dtype) if y is not None else 0), _c_float(y_scale),
        _ptr(weight), _c_int(dtype_code(weight.dtype)), _c_float(eps), _ptr(out),
        _c_int(dtype_code(out.dtype)), _c_float(out_scale), _ptr(rows), _c_int(n), _c_int(H), _stream()),
        "add_rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, interleave: int = 0) -> torch.Tensor:
    """``silu(gate) * up``.  ``interleave`` 0: ``gate_up = [gate | up]``; 8: eight
    gate columns, then the eight up columns of the same features, and so on."""
    T, I2 = gate_up.shape
    I = I2 // 2
    _contig(gate_up, "gate_up")
    if out is None:
        out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    _check(library().exl3_silu_mul(_ptr(gate_up), _ptr(out), _c_int(dtype_code(gate_up.dtype)), _c_int(T),
                                   _c_int(I), _c_int(interleave), _stream()), "silu_mul")
    return out


def rotary_table(frequencies: torch.Tensor) -> torch.Tensor:
    """Float64 frequencies as the kernels take them: float32 ``[2, n]``, row 0 the frequencies rounded to
    float32, row 1 what the rounding lost, so that the angle ``position * frequency`` keeps its accuracy at
    large positions.  A plain float32 ``[n]`` table is taken too (no second term)."""
    f = frequencies.to(torch.float64)
    hi = f.to(torch.float32)
    lo = (f - hi.to(torch.float64)).to(torch.float32)
    return torch.stack([hi, lo]).contiguous()


def _rotary_rows(inv_freq: torch.Tensor, rot: int, what: str):
    """The frequency table's pointers: (frequencies, their float32 remainders or null)."""
    if inv_freq.dtype != torch.float32 or inv_freq.numel() not in (rot // 2, rot) or \
            (inv_freq.numel() == rot and inv_freq.dim() != 2):
        raise KernelLibraryError(f"{what}: inv_freq must be float32 with rot / 2 entries, or [2, rot / 2] "
                                 "(see rotary_table)")
    _contig(inv_freq, "inv_freq")
    if inv_freq.dim() == 2 and inv_freq.shape[0] == 2:
        return _ptr(inv_freq[0]), _ptr(inv_freq[1])
    return _ptr(inv_freq), _c_void_p(0)


def rope_kv_write(qkv: torch.Tensor, inv_freq: torch.Tensor, rot: int, pos_scale: float,
                  tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                  k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], heads: int, kv_heads: int,
                  head_dim: int, page: int, write_kv: bool) -> None:
    """Rotates q and k inside ``qkv`` and writes rotated k and v to the cache."""
    T = qkv.shape[0]
    _contig(qkv, "qkv")
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelLibraryError("rope_kv_write: qkv width does not match the head counts")
    hi, lo = _rotary_rows(inv_freq, rot, "rope_kv_write") if rot else (_c_void_p(0), _c_void_p(0))
    if write_kv and (k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype):
        raise KernelLibraryError("rope_kv_write: cache and activations differ in element type")
    _check(library().exl3_rope_kv_write(
        _ptr(qkv), _c_int(dtype_code(qkv.dtype)), hi, lo, _c_int(rot), _c_float(pos_scale),
        _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), _c_int(block_table.stride(0)),
        _ptr(k_pool) if write_kv else _c_void_p(0), _ptr(v_pool) if write_kv else _c_void_p(0), _c_int(T),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(1 if write_kv else 0),
        _stream()), "rope_kv_write")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` on the CUDA cores, float32 accumulation in K order."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != w.dtype or (bias is not None and bias.dtype != w.dtype):
        raise KernelLibraryError("gemm: x, w and bias must share an element type")
    _contig(x, "x")
    _contig(w, "w")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemm_simt(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(x.dtype)),
                                    _c_int(dtype_code(out.dtype)), _c_int(M), _c_int(N), _c_int(K),
                                    _stream()), "gemm_simt")
    return out


GEMV_MAX_ROWS = 16


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
              out: Optional[torch.Tensor] = None, gated: bool = False) -> torch.Tensor:
    """``x @ w.T (+ bias)`` for at most 16 rows of x, weights read once.  With
    ``gated`` the rows of w are eight gate rows then the eight up rows of the
    same features, repeated, and ``silu(gate) * up`` comes out (N / 2 wide)."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemv: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemv_bf16: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemv_bf16(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)),
                                    _c_int(M), _c_int(N), _c_int(K), _c_int(1 if gated else 0), _stream()),
           "gemv_bf16")
    return out


def gemv_bf16_normed(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                     gated: bool = False, scale=None, resid=None):
    """``gemv_bf16`` as one or both sides of a norm that is no kernel of its own (see gemv_bf16.cuh).

    ``scale = (ss, eps, width)``: ``x`` is the ``x_raw`` of a producing call; results are multiplied per batch row
    by ``rsqrt(ss.sum(1) / width + eps)`` before bias and gating.
    ``resid = (h, rho, norm_w)``: nothing is returned as output; ``h += result * rho`` in place (float32), and
    ``(x_raw, ss)`` is returned: ``h * norm_w`` as bfloat16 and the blocks' sums of squares ``[16, ceil(N/16)]``."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemv_bf16_normed: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemv_bf16_normed: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemv_bf16_normed: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    if resid is not None:
        if gated:
            raise KernelLibraryError("gemv_bf16_normed: the gated epilogue does not write into the residual")
        h, rho, norm_w = resid
        if h.dtype != torch.float32 or tuple(h.shape) != (M, N) or tuple(norm_w.shape) != (N,):
            raise KernelLibraryError(f"gemv_bf16_normed: h {tuple(h.shape)} / norm weight {tuple(norm_w.shape)} "
                                     f"do not fit an output of {(M, N)}")
        _contig(h, "h")
        _contig(norm_w, "norm_w")
        x_raw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ss_out = torch.empty((16, (N + 15) // 16), dtype=torch.float32, device=x.device)
        _check(library().exl3_gemv_bf16_normed(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(None), _c_int(DT_BF16), _c_int(M), _c_int(N), _c_int(K), _c_int(2),
            _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(h), _c_float(rho), _ptr(norm_w),
            _c_int(dtype_code(norm_w.dtype)), _ptr(x_raw), _ptr(ss_out), _stream()), "gemv_bf16_normed")
        return x_raw, ss_out
    out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemv_bf16_normed(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)), _c_int(M), _c_int(N), _c_int(K),
        _c_int(1 if gated else 0), _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(None),
        _c_float(0.0), _ptr(None), _c_int(DT_BF16), _ptr(None), _ptr(None), _stream()), "gemv_bf16_normed")
    return out


SKINNY_MAX_ROWS = 128


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                gated: bool = False, scale=None, resid=None, split: int = 0, out: Optional[torch.Tensor] = None,
                tiles: int = 0):
    """``x @ w.T (+ bias)`` for up to 128 rows of x on the tcgen05 tensor cores with the weights read once (the
    weights are the 128-row operand, the batch the narrow one; see gemm_skinny.cu).  ``gated``, ``scale`` and
    ``resid`` as in ``gemv_bf16_normed``; the sums of squares are ``[rows, blocks]`` with any number of rows from
    M up.  ``split``: blocks that share one tile's K range, 0 for the kernel's own choice from N and K;
    ``tiles``: 128-row tiles of w per block (1 or 2; changes no result), 0 for the kernel's choice."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm_skinny: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_skinny: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemm_skinny: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    lib = library()
    if resid is not None:
        if gated:
            raise KernelLibraryError("gemm_skinny: the gated epilogue does not write into the residual")
        h, rho, norm_w = resid
        if h.dtype != torch.float32 or tuple(h.shape) != (M, N) or tuple(norm_w.shape) != (N,):
            raise KernelLibraryError(f"gemm_skinny: h {tuple(h.shape)} / norm weight {tuple(norm_w.shape)} "
                                     f"do not fit an output of {(M, N)}")
        _contig(h, "h")
        _contig(norm_w, "norm_w")
        x_raw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ss_out = torch.empty((M, (N + 15) // 16), dtype=torch.float32, device=x.device)
        _check(lib.exl3_gemm_skinny(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(None), _c_int(DT_BF16), _c_int(M), _c_int(N), _c_int(K), _c_int(2),
            _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(h), _c_float(rho), _ptr(norm_w),
            _c_int(dtype_code(norm_w.dtype)), _ptr(x_raw), _ptr(ss_out), _c_int(split), _c_int(tiles), _stream()), "gemm_skinny")
        return x_raw, ss_out
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    elif tuple(out.shape) != (M, N // 2 if gated else N) or not out.is_contiguous():
        raise KernelLibraryError(f"gemm_skinny: out must be contiguous {(M, N // 2 if gated else N)}")
    _check(lib.exl3_gemm_skinny(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)), _c_int(M), _c_int(N), _c_int(K),
        _c_int(1 if gated else 0), _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(None),
        _c_float(0.0), _ptr(None), _c_int(DT_BF16), _ptr(None), _ptr(None), _c_int(split), _c_int(tiles), _stream()),
        "gemm_skinny")
    return out


def gemm_skinny_status() -> int:
    """0, or the code a skinny GEMM left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_gemm_skinny_status())


def gemm_skinny_split(N: int, K: int) -> int:
    """The number of K cuts ``gemm_skinny`` chooses for a weight matrix ``[N, K]``."""
    return int(library().exl3_gemm_skinny_split(_c_int(N), _c_int(K)))


def gemm_pair(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
              out_dtype: torch.dtype = torch.bfloat16, gated: bool = False, scale=None, resid=None,
              out: Optional[torch.Tensor] = None):
    """``x @ w.T (+ bias)`` in bfloat16 for many rows of x, two blocks of a cluster as one tensor core
    (tcgen05.mma.cta_group::2, tiles of 256 x 256; see gemm_pair.cu).  ``gated``, ``scale`` and ``resid`` as in
    ``gemm_skinny``; with ``resid`` the sums of squares come back as ``[M, tiles of 256 columns]`` and the product
    is added to the residual without being rounded to bfloat16 first."""
    if out_dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_pair: the output is bfloat16")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm_pair: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_pair: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemm_pair: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    lib = library()
    if resid is not None:
        if gated:
            raise KernelLibraryError("gemm_pair: the gated epilogue does not write into the residual")
        h, rho, norm_w = resid
        if h.dtype != torch.float32 or tuple(h.shape) != (M, N) or tuple(norm_w.shape) != (N,):
            raise KernelLibraryError(f"gemm_pair: h {tuple(h.shape)} / norm weight {tuple(norm_w.shape)} "
                                     f"do not fit an output of {(M, N)}")
        _contig(h, "h")
        _contig(norm_w, "norm_w")
        x_raw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ss_out = torch.empty((M, int(lib.exl3_gemm_pair_ss_blocks(_c_int(N)))), dtype=torch.float32, device=x.device)
        _check(lib.exl3_gemm_pair(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(None), _c_int(M), _c_int(N), _c_int(K), _c_int(2), _ptr(ss_in),
            _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(h), _c_float(rho), _ptr(norm_w),
            _c_int(dtype_code(norm_w.dtype)), _ptr(x_raw), _ptr(ss_out), _stream()), "gemm_pair")
        return x_raw, ss_out
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=torch.bfloat16, device=x.device)
    elif tuple(out.shape) != (M, N // 2 if gated else N) or not out.is_contiguous() or out.dtype != torch.bfloat16:
        raise KernelLibraryError(f"gemm_pair: out must be contiguous bfloat16 {(M, N // 2 if gated else N)}")
    _check(lib.exl3_gemm_pair(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(1 if gated else 0),
        _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(None), _c_float(0.0), _ptr(None),
        _c_int(DT_BF16), _ptr(None), _ptr(None), _stream()), "gemm_pair")
    return out


def gemm_pair_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], scale, tok_pos: torch.Tensor,
                   tok_seq: torch.Tensor, block_table: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                   rot: int, pos_scale: float, heads: int, kv_heads: int, head_dim: int, page: int,
                   k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], write_kv: bool) -> torch.Tensor:
    """The q/k/v projection of many rows (``gemm_pair``; ``scale`` as there) with the rotary encoding and the
    cache write of ``rope_kv_write`` in its epilogue, for heads of 64 rotated as a whole (``rot`` 64) or not at
    all (0) and pages of 64.  Returns ``[M, (heads + 2 kv_heads) * 64]`` of which only the queries' columns are
    written: the rotated keys and the values are in the cache (when ``write_kv``) and nowhere else."""
    M, K = x.shape
    N = (heads + 2 * kv_heads) * head_dim
    if tuple(w.shape) != (N, K):
        raise KernelLibraryError(f"gemm_pair_rope: x is {tuple(x.shape)}, w is {tuple(w.shape)}, heads need {N} rows")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_pair_rope: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemm_pair_rope: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    if tok_pos.numel() < M or tok_seq.numel() < M:
        raise KernelLibraryError("gemm_pair_rope: a position and a sequence for every row")
    hi, lo = _rotary_rows(inv_freq, rot, "gemm_pair_rope") if rot else (_c_void_p(0), _c_void_p(0))
    pool_rows = 0
    if write_kv:
        if k_pool.dtype != torch.bfloat16 or v_pool.dtype != torch.bfloat16:
            raise KernelLibraryError("gemm_pair_rope: the cache must be bfloat16")
        _contig(k_pool, "k_pool")
        _contig(v_pool, "v_pool")
        pool_rows = k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _check(library().exl3_gemm_pair_rope(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(K), _ptr(ss_in), _c_int(ss_blocks), _c_float(eps),
        _c_float(width), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table) if write_kv else _c_void_p(0),
        _c_int(block_table.stride(0)) if write_kv else _c_int(0), hi, lo, _c_int(rot), _c_float(pos_scale),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _ptr(k_pool) if write_kv else _c_void_p(0),
        _ptr(v_pool) if write_kv else _c_void_p(0), _c_int64(pool_rows), _c_int(1 if write_kv else 0), _stream()),
        "gemm_pair_rope")
    return out


def gemm_pair_efficiency(M: int, N: int, device) -> float:
    """The share of the GPU's pairs of SMs that ``gemm_pair``'s tiles of 256 x 256 keep busy, averaged over its
    rounds of tiles: 72 tiles on 74 pairs 0.97, 32 tiles 0.43, 80 tiles (two rounds, the second nearly empty) 0.54."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    pairs = max(1, sm_count(device) // 2)
    return tiles / float(((tiles + pairs - 1) // pairs) * pairs)


def gemm_pair_status() -> int:
    """0, or the code a paired tensor-core GEMM left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_gemm_pair_status())


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
            gated: bool = False) -> torch.Tensor:
    """``x @ w.T (+ bias)`` in bfloat16 on the tcgen05 tensor cores; with ``gated``
    the rows of w are interleaved in eights and ``silu(gate) * up`` comes out."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm_tc: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_tc: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=torch.bfloat16, device=x.device)
    _check(library().exl3_gemm_tc(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(N), _c_int(K),
                                  _c_int(1 if gated else 0), _stream()), "gemm_tc")
    return out


def gemm_tc_status() -> int:
    """0, or the code a tensor-core GEMM left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_gemm_tc_status())


def gemm_tc_wait_selftest() -> None:
    """Runs a kernel whose mbarrier wait is never satisfied; it must give up and set status 9."""
    _check(library().exl3_gemm_tc_wait_selftest(_stream()), "gemm_tc_wait_selftest")


def attn_tokens_scratch_bytes(T: int, heads: int, head_dim: int, max_splits: int) -> int:
    lib = library()
    lib.exl3_attn_tokens_scratch_bytes.restype = _c_size_t
    return int(lib.exl3_attn_tokens_scratch_bytes(_c_int(T), _c_int(heads), _c_int(head_dim), _c_int(max_splits)))


def attn_tokens(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor,
                v_pool: torch.Tensor, block_table: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                T: int, heads: int, kv_heads: int, head_dim: int, page: int, window: int, scale: float,
                split_keys: int, max_splits: int, scratch: Optional[torch.Tensor]) -> torch.Tensor:
    """Attention of T query tokens over the paged cache (see attention_simt.cu)."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelLibraryError("attn_tokens: q, cache and out differ in element type")
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _check(library().exl3_attn_tokens(
        _ptr(q), _c_int64(q_row_stride), _ptr(out), _c_int(dtype_code(q.dtype)), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), _c_int(block_table.stride(0)), _ptr(tok_pos), _ptr(tok_seq), _c_int(T),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window), _c_float(scale),
        _c_int(split_keys), _c_int(max_splits), _ptr(scratch), _c_size_t(nbytes), _stream()), "attn_tokens")
    return out


def attn_prefill_tc_supported(dtype: torch.dtype, head_dim: int, page: int) -> bool:
    return bool(library().exl3_attn_prefill_tc_supported(_c_int(dtype_code(dtype)), _c_int(head_dim), _c_int(page)))


def attn_prefill_tc_status() -> int:
    """0, or the code a tcgen05 attention kernel left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_attn_prefill_tc_status())


def attn_prefill_tc(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    block_table: torch.Tensor, row_start: torch.Tensor, row_pos0: torch.Tensor,
                    tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, heads: int, kv_heads: int,
                    head_dim: int, page: int, window: int, scale: float, variant: int = 0) -> torch.Tensor:
    """Causal attention of whole prompts on tcgen05 tensor cores (tiles of 128 queries; see
    attention_prefill_tc.cu).  ``k_pool`` / ``v_pool``: one layer's ``[pages, kv_heads, 64, head_dim]``.
    ``variant``: 0 lets the kernel choose by the number of blocks between a tile a block, four blocks per SM (heads
    of 64) and two tiles a block (the list's first with its last, and so on: list the tiles with the most keys
    to visit first); 1, 2 and 3 force one of them (the same numbers every way)."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelLibraryError("attn_prefill_tc: q, cache and out differ in element type")
    _contig(k_pool, "k_pool")
    _contig(v_pool, "v_pool")
    pool_rows = k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2]
    _check(library().exl3_attn_prefill_tc(
        _ptr(q), _c_int64(q_row_stride), _c_int(q.shape[0]), _ptr(out), _ptr(k_pool), _ptr(v_pool),
        _c_int64(pool_rows), _ptr(block_table), _c_int(block_table.stride(0)), _ptr(row_start), _ptr(row_pos0),
        _ptr(tile_seq), _ptr(tile_q0), _c_int(n_tiles), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
        _c_int(page), _c_int(window), _c_float(scale), _c_int(variant), _stream()), "attn_prefill_tc")
    return out


_SM_COUNT: dict = {}


def sm_count(device: torch.device) -> int:
    """Streaming multiprocessors of ``device`` (looked up once)."""
    key = torch.device(device).index or 0
    n = _SM_COUNT.get(key)
    if n is None:
        n = _SM_COUNT[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return n


ATTN_DECODE_MAX_CHUNKS = 256      # chunks of one (token, kv head) that attn_decode takes


def attn_decode_supported(dtype: torch.dtype, T: int, heads: int, kv_heads: int, head_dim: int, page: int,
                          split_keys: int, max_splits: int) -> bool:
    return bool(library().exl3_attn_decode_supported(
        _c_int(dtype_code(dtype)), _c_int(T), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page),
        _c_int(split_keys), _c_int(max_splits)))


def attn_decode_status() -> int:
    """0, or the code the decode attention kernel left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_attn_decode_status())


def attn_decode(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                block_table: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor, T: int, heads: int,
                kv_heads: int, head_dim: int, page: int, window: int, scale: float, split_keys: int,
                max_splits: int, scratch: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor] = None,
                rot: int = 0, pos_scale: float = 1.0, write_new: bool = False, head_split: int = 1,
                in_block: int = 0, twins: int = 1) -> torch.Tensor:
    """Attention of T query tokens over the paged cache on the tensor cores (see attention_decode.cu);
    arguments and scratch as ``attn_tokens``.  With ``write_new``, ``q`` is the fused q|k|v output of the
    projection, every token is its sequence's only new one and the cache holds the positions before it: the
    kernel adds the token's own key and value to its softmax and writes them to the cache.  With ``rot`` equal to
    ``head_dim`` it applies the half-split rotary encoding (``inv_freq``: head_dim / 2 float32 frequencies, or a ``rotary_table``) to
    the queries and the new key.  ``head_split`` n (a divisor of the query heads per kv head) makes n groups of work
    of a kv head's query heads: n times the work items, each merge an n-th of the size; changes no result.
    ``in_block`` 1 (or True): one block per (token, group of heads), whose four warps take the item's chunks
    (``max_splits`` at most 4) and merge them in shared memory; 2: a cluster of two blocks per item (at most 8
    chunks; the first block merges and reads the second one's records out of its shared memory): no scratch, no
    tickets; results differ from the other way's by rounding (another order of the same sums).  ``twins`` 2 (with
    ``in_block`` 1 or 2, an even ``head_split`` and groups of up to 8 heads): a block takes two groups of query heads
    of a kv head, whose warps walk the same pages out of the same rings; changes no result."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelLibraryError("attn_decode: q, cache and out differ in element type")
    _contig(k_pool, "k_pool")
    _contig(v_pool, "v_pool")
    hi = lo = _c_void_p(0)
    if rot:
        if inv_freq is None:
            raise KernelLibraryError("attn_decode: rot needs inv_freq")
        hi, lo = _rotary_rows(inv_freq, rot, "attn_decode")
    pool_rows = k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2]
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _check(library().exl3_attn_decode(
        _ptr(q), _c_int64(q_row_stride), _ptr(out), _ptr(k_pool), _ptr(v_pool), _c_int64(pool_rows),
        _ptr(block_table), _c_int(block_table.stride(0)), _ptr(tok_pos), _ptr(tok_seq), _c_int(T), _c_int(heads),
        _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window), _c_float(scale), _c_int(split_keys),
        _c_int(max_splits), _ptr(scratch), _c_size_t(nbytes), hi, lo, _c_int(rot),
        _c_float(pos_scale), _c_int(1 if write_new else 0), _c_int(head_split), _c_int(int(in_block)),
        _c_int(int(twins)), _stream()), "attn_decode")
    return out


def check_status() -> None:
    """Raises if a kernel with bounded waits (the tcgen05 GEMMs and attention, the TMA decode attention) gave up
    on one since the last call: its results are then not to be trusted.  Reads four flags from the device, so
    it waits for the work launched so far; call it where the host waits anyway."""
    gave_up = [name for name, fn in (("gemm_tc", gemm_tc_status), ("gemm_skinny", gemm_skinny_status),
                                     ("gemm_pair", gemm_pair_status),
                                     ("attn_prefill_tc", attn_prefill_tc_status),
                                     ("attn_decode", attn_decode_status)) if fn()]
    if gave_up:
        raise KernelLibraryError("a bounded wait ran out in " + ", ".join(gave_up) +
                                 ": a copy or a tensor-core product did not complete in time")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    R, V = logits.shape
    if logits.dtype != torch.float32:
        raise KernelLibraryError("argmax: logits must be float32")
    _contig(logits, "logits")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    lib = library()
    lib.exl3_argmax_scratch_bytes.restype = _c_size_t
    need = int(lib.exl3_argmax_scratch_bytes(_c_int(R), _c_int(V)))
    scratch = torch.empty(need // 4, dtype=torch.float32, device=logits.device) if need else None
    _check(lib.exl3_argmax(_ptr(logits), _ptr(out), _c_int(R), _c_int(V), _ptr(scratch), _c_size_t(need),
                           _stream()), "argmax")
    return out


def sample_filtered_cap() -> int:
    """The most candidates the device sampler ranks (``top_k`` above it is the host sampler's)."""
    return int(library().exl3_sample_filtered_cap())


def sample_filtered(logits: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The reference's sampler on the device.  ``rows``: float64 ``[R, 5]`` on the device: temperature (<= 0:
    greedy), top_k (0: off), top_p, min_p and the row's uniform number in [0, 1)."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or rows.dtype != torch.float64 or tuple(rows.shape) != (R, 5):
        raise KernelLibraryError("sample_filtered: logits [R, V] must be float32 and rows [R, 5] float64")
    _contig(logits, "logits")
    _contig(rows, "rows")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _check(library().exl3_sample_filtered(_ptr(logits), _ptr(rows), _ptr(out), _c_int(R), _c_int(V), _stream()),
           "sample_filtered")
    return out


def sample_penalties(logits: torch.Tensor, counts: torch.Tensor, params: torch.Tensor) -> None:
    """Repetition, presence and frequency penalties, in place.  ``counts``: int64 ``[R]`` on the device, the
    addresses of the rows' int32 ``[V]`` token counts (0: the row has none); ``params``: float32 ``[R, 3]``."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or counts.dtype != torch.int64 or params.dtype != torch.float32 or \
            counts.numel() != R or tuple(params.shape) != (R, 3):
        raise KernelLibraryError("sample_penalties: logits float32 [R, V], counts int64 [R], params float32 [R, 3]")
    _contig(logits, "logits")
    _contig(params, "params")
    _check(library().exl3_sample_penalties(_ptr(logits), _c_int(R), _c_int(V), _ptr(counts), _ptr(params),
                                           _stream()), "sample_penalties")


def sample_count(counts: torch.Tensor, ids: torch.Tensor, vocab: int) -> None:
    """Adds each row's chosen token (``ids`` int32 ``[R]``) to its counts (``counts`` as in ``sample_penalties``)."""
    if counts.dtype != torch.int64 or ids.dtype != torch.int32 or counts.numel() != ids.numel():
        raise KernelLibraryError("sample_count: counts int64 [R] and ids int32 [R]")
    _check(library().exl3_sample_count(_ptr(counts), _ptr(ids), _c_int(ids.numel()), _c_int(vocab), _stream()),
           "sample_count")
