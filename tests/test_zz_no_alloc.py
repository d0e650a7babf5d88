"""The allocation-free abs-max entry point, called through its exported C symbol.

Who needs it: callers that may not allocate device memory when they need the norm (frozen allocators of
real-time loops, plugins inside a host that owns all device memory, code inside allocator callbacks).
The test checks two consecutive calls against the regular (allocating) ``ops.absmax`` -- exact equality,
the tolerance the other abs-max tests use -- plus the size limit and the argument checks.  Collected last
on purpose: a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from gradient_compression_b200 import build

    lib = ctypes.CDLL(build.build_cuda())
    fn = lib.gcb200_absmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.gcb200_noalloc_strerror.restype = ctypes.c_char_p
    lib.gcb200_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def test_noalloc_absmax_matches_regular_entry_point_twice_in_a_row():
    from gradient_compression_b200 import ops

    lib, fn = _lib()
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(123)
    inputs = [torch.randn((1 << 22) + 5, generator=g).cuda() * 3e-3, torch.randn(4099, generator=g).cuda() * 7.0]
    out = torch.full((1,), -1.0, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for x in inputs:                                    # two calls back to back share the scratch array
        rc = fn(x.data_ptr(), x.numel(), out.data_ptr(), stream)
        assert rc == 0, lib.gcb200_noalloc_strerror(rc)
        expect = ops.absmax(x)
        torch.cuda.synchronize()
        assert float(out) == float(expect) == float(x.abs().max())
    # an unaligned input pointer and n = 0
    y = inputs[1][1:]
    assert fn(y.data_ptr(), y.numel(), out.data_ptr(), stream) == 0
    assert float(out) == float(y.abs().max())
    assert fn(None, 0, out.data_ptr(), stream) == 0
    assert float(out) == 0.0


def test_noalloc_rejects_oversize_and_bad_arguments():
    lib, fn = _lib()
    torch.cuda.set_device(0)
    out = torch.zeros(1, device="cuda")
    x = torch.zeros(8, device="cuda")
    rc = fn(x.data_ptr(), (1 << 30) + 1, out.data_ptr(), None)
    assert rc == -2 and b"exceeds" in lib.gcb200_noalloc_strerror(rc)
    assert fn(x.data_ptr(), 8, None, None) == -1
    assert fn(None, 8, out.data_ptr(), None) == -1
    assert fn(x.data_ptr(), -1, out.data_ptr(), None) == -1
