"""The argmax entry point that brings its own scratch memory, for callers that
may not allocate on the device (a host that owns all GPU memory through its own
pool, a thread that must stay out of the driver's allocator, plug-in code that
only gets buffers handed in).  It is called here through its exported C symbol,
with nothing but the caller's input and output buffers, twice in a row, and
must agree with the ordinary entry point, which is given scratch by its caller.

This file sorts last on purpose: if it fails, a run that stops at the first
failure has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(lib, logits, out):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.exl3_argmax_static(ctypes.c_void_p(logits.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                  ctypes.c_int(logits.shape[0]), ctypes.c_int(logits.shape[1]), stream)


def test_argmax_static_matches_the_ordinary_entry_point_twice_in_a_row():
    from exl3_server_b200.ops import kernels as K
    from exl3_server_b200.ops.lib import library
    lib = library()
    lib.exl3_argmax_static.restype = ctypes.c_int
    torch.cuda.set_device(0)
    g = torch.Generator(device=DEV).manual_seed(11)
    # two calls in a row with different sizes and contents: the second must not see the first's leftovers
    for rows, vocab in ((7, 122753), (64, 5000), (3, 300)):
        logits = torch.randn(rows, vocab, device=DEV, generator=g)
        logits[0, vocab - 1] = 99.0
        logits[rows - 1, 0] = 98.0
        logits[rows // 2, vocab // 3] = logits[rows // 2].max() + 1.0
        logits[rows // 2, vocab // 3 + 1] = logits[rows // 2, vocab // 3]          # a tie: the first wins
        want = K.argmax(logits)
        out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        assert _call_static(lib, logits, out) == 0, lib.exl3_last_error()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
        assert out[0] == vocab - 1 and out[rows - 1] == 0 and out[rows // 2] == vocab // 3


def test_argmax_static_refuses_what_its_scratch_cannot_hold():
    from exl3_server_b200.ops.lib import library
    lib = library()
    lib.exl3_argmax_static.restype = ctypes.c_int
    lib.exl3_last_error.restype = ctypes.c_char_p
    out = torch.zeros(65, dtype=torch.int32, device=DEV)
    too_many_rows = torch.zeros(65, 8, device=DEV)
    assert _call_static(lib, too_many_rows, out) != 0
    assert b"at most 64 rows" in lib.exl3_last_error()
    too_wide = torch.zeros(1, 524289, device=DEV)
    assert _call_static(lib, too_wide, out) != 0
    assert b"exceed the built-in scratch" in lib.exl3_last_error()
