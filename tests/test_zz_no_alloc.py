"""The allocation-free C entry point ``sb200_sumsq_bf16_noalloc``.

It is meant for callers that may not allocate device memory (health probes that
must not enter the caching allocator, out-of-memory handlers, embedders with a
fixed memory budget): its scratch lives in a fixed array inside the library.  The test calls it through its exported C symbol with
ctypes -- inputs and the output scalar are ordinary caller-owned device tensors --
and checks it against the regular operator (``ops.sum_of_squares``, which takes
its scratch from the allocator) on two consecutive calls, because all calls share
one scratch array that keeps the previous call's contents.  The file name sorts
last on purpose: a run that stops at the first failure has then already executed
every other test.
"""

import ctypes

import pytest
import torch

from speculators_b200 import ops
from speculators_b200.ops import _build

pytestmark = pytest.mark.gpu

MAX_ELEMENTS = 65536 * 16384


def _entry():
    ops.native()  # builds the shared object if needed
    lib = ctypes.CDLL(str(_build.LIB))
    fn = lib.sb200_sumsq_bf16_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.sb200_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _call(fn, x, out, accumulate=False):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(x.data_ptr(), x.numel(), out.data_ptr(), int(accumulate), ctypes.c_void_p(stream))


def test_two_calls_in_a_row_match_the_allocating_operator():
    torch.cuda.set_device(0)
    lib, fn = _entry()
    torch.manual_seed(0)
    # second call is shorter than the first: stale partials of call 1 must not leak in
    sizes = [3 * 65536 + 12345, 65536 + 7]
    for n in sizes:
        x = torch.randn(n, device="cuda").to(torch.bfloat16)
        got = torch.full((1,), -1.0, device="cuda")
        want = torch.zeros(1, device="cuda")
        assert _call(fn, x, got) == 0, lib.sb200_noalloc_last_error()
        ops.sum_of_squares(x, want)
        torch.cuda.synchronize()
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-2)
        torch.testing.assert_close(got[0], x.float().pow(2).sum(), rtol=1e-4, atol=1e-2)
    # accumulate mode adds onto the existing value
    assert _call(fn, x, got, accumulate=True) == 0
    torch.cuda.synchronize()
    torch.testing.assert_close(got, 2 * want, rtol=1e-4, atol=2e-2)


def test_empty_input_and_rejections():
    torch.cuda.set_device(0)
    lib, fn = _entry()
    out = torch.full((1,), 5.0, device="cuda")
    empty = torch.empty(0, device="cuda", dtype=torch.bfloat16)
    assert fn(None, 0, out.data_ptr(), 0, None) == 0
    torch.cuda.synchronize()
    assert float(out) == 0.0
    x = torch.ones(8, device="cuda", dtype=torch.bfloat16)
    assert fn(x.data_ptr(), MAX_ELEMENTS + 1, out.data_ptr(), 0, None) == -2  # nothing is launched
    assert b"exceeds" in lib.sb200_noalloc_last_error()
    assert fn(x.data_ptr(), 8, None, 0, None) == -1
    assert fn(None, 8, out.data_ptr(), 0, None) == -1
    del empty
