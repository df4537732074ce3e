"""The allocation-free entry point ``elfa_sumsq_static``.

Some hosts that load the library may not allocate device memory (another runtime owns the pool,
or allocation is forbidden where they call from), so they cannot hand ``elfa_sumsq`` its scratch
buffer. This test calls the static-scratch variant through its exported C symbol, twice in a row on
different inputs, and compares it with the regular entry point. It lives in a file that pytest
collects last so that a failure here cannot hide the result of any other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "elfa_b200", "_native", "libelfa_b200.so")


def _symbols():
    dll = ctypes.CDLL(LIB)
    f = dll.elfa_sumsq_static
    f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    f.restype = ctypes.c_int
    ref = dll.elfa_sumsq
    ref.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    ref.restype = ctypes.c_int
    err = dll.elfa_last_error
    err.restype = ctypes.c_char_p
    return f, ref, err


def test_static_scratch_sumsq_matches_regular_entry_point_twice(cuda_device):
    f, ref, err = _symbols()
    dev = cuda_device
    stream = torch.cuda.current_stream(dev).cuda_stream
    out = torch.zeros(1, dtype=torch.float32, device=dev)
    scal = torch.zeros(4, dtype=torch.float32, device=dev)
    part = torch.zeros(2048, dtype=torch.float32, device=dev)
    torch.manual_seed(11)
    # two calls in a row: the second is smaller and of another dtype, so stale partial sums of the
    # first call would show up if the kernels read slots they did not write
    cases = [(torch.randn(3_000_001, device=dev) * 2.0, 0), (torch.randn(70_001, device=dev).to(torch.bfloat16), 1)]
    for x, typ in cases:
        rc = f(x.data_ptr(), typ, x.numel(), out.data_ptr(), stream)
        assert rc == 0, err()
        rc = ref(x.data_ptr(), typ, x.numel(), part.data_ptr(), scal.data_ptr(), 0, stream)
        assert rc == 0, err()
        torch.cuda.synchronize(dev)
        got, want = out.item(), scal[0].item()
        exact = x.double().pow(2).sum().item()
        assert abs(got - want) <= 1e-4 * abs(want), (got, want)
        assert abs(got - exact) <= 1e-3 * abs(exact), (got, exact)


def test_static_scratch_sumsq_rejects_oversized_and_bad_arguments(cuda_device):
    f, _, err = _symbols()
    out = torch.zeros(1, dtype=torch.float32, device=cuda_device)
    x = torch.ones(8, device=cuda_device)
    too_many = (1024 << 24) + 1
    assert f(x.data_ptr(), 0, too_many, out.data_ptr(), None) == 1
    assert b"ELFA_SUMSQ_STATIC_MAX_ELEMS" in err()
    assert f(x.data_ptr(), 0, 0, out.data_ptr(), None) == 1
    assert f(None, 0, 8, out.data_ptr(), None) == 1
    assert f(x.data_ptr(), 7, 8, out.data_ptr(), None) == 1
