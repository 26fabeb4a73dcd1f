"""The allocation-free entry point, called the way an embedder would: through
its exported C symbol, with caller-owned input and output buffers.

It serves callers that cannot allocate device memory themselves (all memory
already planned by a serving runtime or reserved by a framework allocator,
or a code path where cudaMalloc's device-wide synchronisation is not
acceptable). The result must equal what the library's regular reduce-scatter
produces for a group of one and what plain PyTorch arithmetic in fp32 gives
for ``postscale * (prescale * x)``, and a second call right after the first
must be just as correct, because both share one built-in scratch array that
keeps the first call's leftovers.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_BYTES = 4 << 20
FLOAT32, BFLOAT16 = 7, 10


def _lib():
    import horovod_b200
    path = os.path.join(os.path.dirname(horovod_b200.__file__), "_C.so")
    lib = ctypes.CDLL(path)
    fn = lib.hvd_b200_reducescatter1_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                   ctypes.c_double, ctypes.c_double, ctypes.c_void_p, ctypes.c_char_p,
                   ctypes.c_ulong]
    return fn


def _call(fn, x, out, dtype_id, pre, post):
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), out.data_ptr(), x.numel(), dtype_id, pre, post, stream, err, 256)
    return rc, err.value.decode()


def test_matches_regular_reducescatter_twice_in_a_row():
    import horovod_b200.torch as hvd
    fn = _lib()
    hvd.init()
    try:
        torch.cuda.set_device(0)
        dev = torch.device("cuda", 0)
        torch.manual_seed(0)
        cases = [(torch.float32, FLOAT32, 100003, 0.5, 3.0),
                 (torch.float32, FLOAT32, 1 << 20, 1.0, 0.25),
                 (torch.bfloat16, BFLOAT16, 65537, 2.0, 0.5)]
        for dtype, dtype_id, n, pre, post in cases:
            x = torch.randn(n, device=dev).to(dtype)
            want = hvd.reducescatter(x, op=hvd.Sum, prescale_factor=pre,
                                     postscale_factor=post, name="ref.%d" % n)
            # Two calls back to back on different data: the second sees the
            # scratch exactly as the first left it.
            other = torch.randn(n, device=dev).to(dtype)
            out_a = torch.empty_like(other)
            out_b = torch.empty_like(x)
            rc, msg = _call(fn, other, out_a, dtype_id, pre, post)
            assert rc == 0, msg
            rc, msg = _call(fn, x, out_b, dtype_id, pre, post)
            assert rc == 0, msg
            torch.cuda.synchronize()
            want_a = hvd.reducescatter(other, op=hvd.Sum, prescale_factor=pre,
                                       postscale_factor=post, name="ref2.%d" % n)
            tol = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else \
                dict(rtol=1e-2, atol=1e-2)
            torch.testing.assert_close(out_b, want, **tol)
            torch.testing.assert_close(out_a, want_a, **tol)
            # ... and against the same arithmetic done by PyTorch in fp32.
            torch.testing.assert_close(out_b.float(), _expected(x, pre, post).float(), **tol)
            torch.testing.assert_close(out_a.float(), _expected(other, pre, post).float(), **tol)
    finally:
        hvd.shutdown()


def _expected(x, pre, post):
    """postscale * (prescale * x) with each product rounded to the tensor type,
    which is what the kernel's staging step does."""
    return ((x.float() * pre).to(x.dtype).float() * post).to(x.dtype)


def test_in_place_and_largest_accepted_size():
    """The header allows in == out; and an input of exactly the maximum size
    must be accepted. Both twice in a row, compared with PyTorch arithmetic."""
    fn = _lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    for n, pre, post in [(70001, 0.5, 4.0), (MAX_BYTES // 4, 1.0, 0.125)]:
        for _ in range(2):
            x = torch.randn(n, device=dev)
            want = _expected(x, pre, post)
            rc, msg = _call(fn, x, x, FLOAT32, pre, post)
            assert rc == 0, msg
            torch.cuda.synchronize()
            torch.testing.assert_close(x, want, rtol=1e-6, atol=1e-6)


def test_rejects_oversized_and_bad_arguments():
    fn = _lib()
    torch.cuda.set_device(0)
    x = torch.zeros(16, device="cuda:0")
    err = ctypes.create_string_buffer(256)
    too_many = MAX_BYTES // 4 + 1
    rc = fn(x.data_ptr(), x.data_ptr(), too_many, FLOAT32, 1.0, 1.0, None, err, 256)
    assert rc == 1 and b"larger than the built-in scratch" in err.value
    rc = fn(x.data_ptr(), x.data_ptr(), 16, 99, 1.0, 1.0, None, err, 256)
    assert rc == 2 and b"dtype" in err.value
    rc = fn(None, x.data_ptr(), 16, FLOAT32, 1.0, 1.0, None, err, 256)
    assert rc == 2
    # Counts whose byte size wraps around 64 bits, and dtype ids that would
    # alias a valid one after narrowing to a byte: refused before any launch.
    FLOAT64, INT32 = 8, 4
    rc = fn(x.data_ptr(), x.data_ptr(), 1 << 61, FLOAT64, 1.0, 1.0, None, err, 256)
    assert rc == 1 and b"larger than the built-in scratch" in err.value
    rc = fn(x.data_ptr(), x.data_ptr(), 1 << 62, INT32, 1.0, 1.0, None, err, 256)
    assert rc == 1
    rc = fn(x.data_ptr(), x.data_ptr(), 16, 256 + FLOAT32, 1.0, 1.0, None, err, 256)
    assert rc == 2 and b"dtype" in err.value
    rc = fn(x.data_ptr(), x.data_ptr(), 16, 256, 1.0, 1.0, None, err, 256)
    assert rc == 2
    torch.cuda.synchronize()
