"""A projection ``y = x @ W^T (+ b)`` with W kept in the checkpoint's
``(out, in)`` order (the reference transposes to ``(in, out)`` at load,
src/model.cpp:214-228; the kernels here read rows of W, so no transpose).

Which kernel runs depends only on the element type and the sizes:
float32 goes through the CUDA-core kernel with a fixed order of summation
(the true 32-bit path).  bfloat16 with at most 16 rows streams the weights once
through the tensor-core GEMV (``mma.sync``, weights as the 16-row operand); with
17 to ``SKINNY_ROWS`` rows through the skinny tcgen05 GEMM (weights as the
128-row operand, streamed once by TMA); with more rows (prompts) through the
paired tcgen05 GEMM (two blocks of a cluster on tiles of 256 x 256), when its
tiles fill the GPU (``PAIR_MIN_EFFICIENCY``).  All three take a norm's output in
two pieces and can fold their output into the residual (see ``RawNormed``,
``NormAfter``), so a step has no kernel between its projections but attention and
position encoding.  Products in between (some hundred rows, or a narrow output)
are the library's (cuBLAS through ``torch``), as the reference's are MLX's
(src/model.cpp:549); the gated feed-forward projection, whose epilogue is fused,
never goes to the library.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels as K
from .base import RawNormed


import os

# Rows up to which bfloat16 projections go through the skinny tcgen05 GEMM (17 rows and more; the GEMV below).
SKINNY_ROWS = 64
# Bytes of weights from which the skinny GEMM also takes 1 to 16 rows: its TMA stream is faster than the GEMV's
# per-thread copies once a matrix is large (in chains of one kernel: 53 MB 11.1 against 14.0 us, 134 MB 24.0
# against 27.7 us, 32 MB 8.1 against 7.7 us).  Inside a step the 53 MB matrix gains only from 8 rows on (batch 8
# at the 2B sizes 3.40 -> 3.32 ms, batch 1 1.51 -> 1.53 ms), the larger ones always (8B sizes, batch 1: 3.38 ->
# 3.31 ms).
SKINNY_MIN_BYTES = int(os.environ.get("EXL3_SKINNY_MIN_BYTES", 48 << 20))
SKINNY_MIN_BYTES_FEW_ROWS = int(os.environ.get("EXL3_SKINNY_MIN_BYTES_FEW", 100 << 20))     # fewer than 8 rows
# Above SKINNY_ROWS rows: the least share of the GPU's pairs of SMs that the paired GEMM's tiles must keep busy for
# it to run instead of the library's product (one prompt of 2,048 tokens at the 2B sizes: 0.97 for every projection).
PAIR_MIN_EFFICIENCY = float(os.environ.get("EXL3_PAIR_MIN_EFFICIENCY", 0.7))


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], dtype: torch.dtype):
        if weight.dim() != 2:
            raise ValueError(f"Linear: weight must be 2-dimensional, got {tuple(weight.shape)}")
        self.weight = weight.to(dtype).contiguous()
        self.bias = None if bias is None else bias.to(dtype).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.dtype = dtype

    def _streaming_kernel(self, rows: int):
        """The kernel of this library that takes ``rows`` rows and the norm's pieces: the GEMV, the skinny GEMM, the
        paired GEMM, or None (float32, sizes they refuse, or too few tiles for the paired one)."""
        if self.dtype != torch.bfloat16 or self.in_features % 8 != 0:
            return None
        if rows <= K.GEMV_MAX_ROWS and self.weight.numel() * 2 < (SKINNY_MIN_BYTES if rows >= 8
                                                                    else SKINNY_MIN_BYTES_FEW_ROWS):
            return K.gemv_bf16_normed
        if rows <= SKINNY_ROWS:
            return K.gemm_skinny
        if self.out_features % 8 == 0 and \
                K.gemm_pair_efficiency(rows, self.out_features, self.weight.device) >= PAIR_MIN_EFFICIENCY:
            return K.gemm_pair
        return None

    def __call__(self, x, out_dtype: Optional[torch.dtype] = None, then=None) -> Optional[torch.Tensor]:
        """``x``: a tensor, or a ``RawNormed`` (a norm's output in two pieces: the weight-streaming kernels apply
        the missing factor per row to their results; other paths materialise it first).
        ``then``: a ``NormAfter`` offer; taken when one of this library's bfloat16 kernels runs and the output is
        as wide as the residual: its blocks add the output to the residual and leave the pieces of the next norm's
        output.  Returns None then."""
        out_dtype = out_dtype or self.dtype
        M = x.shape[0]
        fast = self.in_features % 8 == 0
        kernel = self._streaming_kernel(M)
        if kernel is K.gemm_pair and out_dtype != torch.bfloat16:
            kernel = None                       # float32 results for many rows: below
        scale = None
        if isinstance(x, RawNormed):
            if kernel is not None:
                scale, x = (x.ss, x.eps, float(x.width)), x.x_raw
            else:
                x = x.materialize()
        if self.dtype == torch.float32:
            return K.gemm_simt(x, self.weight, self.bias, torch.float32)
        if kernel is not None:
            if (then is not None and out_dtype == torch.bfloat16 and hasattr(then.norm, "fuse_args")
                    and then.stream.pending is None and tuple(then.stream.h.shape) == (M, self.out_features)):
                norm_w, eps, width = then.norm.fuse_args()
                x_raw, ss = kernel(x, self.weight, self.bias, torch.bfloat16, scale=scale,
                                   resid=(then.stream.h, then.scale, norm_w))
                then.stream.normed = (then.norm, RawNormed(x_raw, ss, eps, width))
                then.done = True
                return None
            if scale is None and kernel is K.gemv_bf16_normed:
                return K.gemv_bf16(x, self.weight, self.bias, out_dtype)
            return kernel(x, self.weight, self.bias, out_dtype, scale=scale)
        if out_dtype == torch.bfloat16 and fast:
            return torch.nn.functional.linear(x, self.weight, self.bias)
        if fast:
            # float32 results for many rows (logits at many positions): the skinny GEMM in groups of 128 rows
            # keeps float32 accumulators end to end
            out = torch.empty((M, self.out_features), dtype=out_dtype, device=x.device)
            for m0 in range(0, M, K.SKINNY_MAX_ROWS):
                m1 = min(M, m0 + K.SKINNY_MAX_ROWS)
                K.gemm_skinny(x[m0:m1], self.weight, self.bias, out_dtype, out=out[m0:m1])
            return out
        return K.gemm_simt(x, self.weight, self.bias, out_dtype)

    def heads_rotated_and_cached(self, x, heads: int, kv_heads: int, head_dim: int, page: int, rotation, batch, kv):
        """For a weight that is a q/k/v projection: the product of many rows with the rotary encoding and the
        cache write in its epilogue (``rotation``: a position part's ``fused_rotation``; keys and values go to
        ``kv`` when it owns its pages).  Returns ``[rows, (heads + 2 kv_heads) * head_dim]`` with the queries'
        columns written, or None when the sizes are not the paired GEMM's with that epilogue (heads and pages of
        64, enough rows): the caller then projects, rotates and stores in separate steps."""
        if rotation is None or head_dim != 64 or page != 64 or kv is None:
            return None
        inv_freq, rot, pos_scale = rotation
        if rot not in (0, head_dim) or self._streaming_kernel(x.shape[0]) is not K.gemm_pair:
            return None
        scale = None
        if isinstance(x, RawNormed):
            scale, x = (x.ss, x.eps, float(x.width)), x.x_raw
        write = bool(kv.owns)
        return K.gemm_pair_rope(x, self.weight, self.bias, scale, batch.tok_pos, batch.tok_seq, kv.block_table,
                                inv_freq, rot, pos_scale, heads, kv_heads, head_dim, page,
                                kv.k if write else None, kv.v if write else None, write)

    def streams_weights(self, rows: int) -> bool:
        """Whether ``rows`` rows of input go through a kernel that reads the weights once."""
        return self._streaming_kernel(rows) is not None

    def fuses_gate(self) -> bool:
        """Whether ``gated`` can run: bfloat16 with sizes the fused kernels take."""
        return self.dtype == torch.bfloat16 and self.in_features % 8 == 0 and self.out_features % 16 == 0

    def gated(self, x: torch.Tensor) -> torch.Tensor:
        """For a weight whose rows are eight gate rows, then the eight up rows
        of the same features, and so on: ``silu(gate) * up`` in the projection's
        own epilogue, so the gate/up product never goes to memory.  Up to 16 rows:
        the weight-streaming GEMV; up to ``SKINNY_ROWS``: the skinny tcgen05 GEMM; more: the paired tcgen05 GEMM,
        or the one-block tcgen05 GEMM when the paired one's tiles would leave the GPU half empty."""
        kernel = self._streaming_kernel(x.shape[0])
        if isinstance(x, RawNormed):
            if kernel is not None:
                return kernel(x.x_raw, self.weight, self.bias, self.dtype, gated=True,
                              scale=(x.ss, x.eps, float(x.width)))
            x = x.materialize()
        if kernel is K.gemv_bf16_normed:
            return K.gemv_bf16(x, self.weight, self.bias, self.dtype, gated=True)
        if kernel is not None:
            return kernel(x, self.weight, self.bias, self.dtype, gated=True)
        return K.gemm_tc(x, self.weight, self.bias, gated=True)

    def weight_bytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        if self.bias is not None:
            n += self.bias.numel() * self.bias.element_size()
        return n
