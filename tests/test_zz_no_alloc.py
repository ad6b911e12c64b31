"""The allocation-free column sum (``rb_colsum_noalloc``), called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need a kernel — a host
application that has handed the whole GPU to a frozen memory pool, or a latency-critical loop that must
never hit ``cudaMalloc``.  For them the library carries its own scratch; this test checks that the
entry point gives the same sums as the regular one (which takes a caller-provided workspace), twice in
a row on the same stream (the built-in scratch is shared by all calls, so the second call must not see
leftovers of the first), and that it refuses inputs wider than its built-in scratch.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_colsum_matches_regular_entry_point_twice():
    from renee_b200.ops import cuda as cu
    lib = cu.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    fn = lib.rb_colsum_noalloc
    fn.restype = ctypes.c_int
    max_cols = lib.rb_colsum_noalloc_max_cols()
    assert max_cols == 8192
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for (rows, N, dt) in ((777, 2304, torch.bfloat16), (64, 8192, torch.float32)):
        torch.manual_seed(rows)
        x = torch.randn(rows, N, device=dev).to(dt)
        want = torch.empty(N, device=dev, dtype=dt)
        cu.colsum(x, want)                                    # regular entry point, caller-provided workspace
        for _ in range(2):                                    # two calls in a row share the built-in scratch
            got = torch.full((N,), 123.0, device=dev, dtype=dt)
            rc = fn(ctypes.c_int(cu.DT[dt]), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(got.data_ptr()),
                    ctypes.c_int(rows), ctypes.c_int(N), stream)
            assert rc == 0
            torch.cuda.synchronize()
            tol = dict(rtol=3e-2, atol=1e-1) if dt != torch.float32 else dict(rtol=1e-4, atol=1e-3)
            torch.testing.assert_close(got.float(), want.float(), **tol)
            torch.testing.assert_close(got.float(), x.float().sum(0), **tol)
    # wider than the built-in scratch: refused, nothing launched
    x = torch.zeros(8, max_cols + 8, device=dev)
    out = torch.zeros(max_cols + 8, device=dev)
    rc = fn(ctypes.c_int(0), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(8),
            ctypes.c_int(max_cols + 8), stream)
    assert rc == -10
    # an unknown dtype code is refused before anything is queued on the stream
    rc = fn(ctypes.c_int(7), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(8),
            ctypes.c_int(64), stream)
    assert rc == -1
