"""The allocation-free entry point ``ob200_two_sided_apply_noalloc``.

Some callers of the preconditioner product P = L G R cannot allocate device memory when they
need it: code inside a region where the device heap is frozen, plug-ins inside a host process
that owns all device memory, latency-critical loops.  For them the library exports one C
function whose m x n intermediate lives in a fixed array inside the library.  This test calls
that function through its exported C symbol (ctypes, raw device pointers, nothing from torch's
allocator on its path) and checks it against the regular, allocating entry point on two calls
in a row; the second call reuses the scratch that the first one left dirty, with a different
shape, so stale contents would show.  The file is named to be collected last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMS = 1 << 20


def _lib_and_ext():
    from optimizers_b200.ops import build

    ext = build.load()
    lib = ctypes.CDLL(ext.__file__)
    fn = lib.ob200_two_sided_apply_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.ob200_noalloc_strerror.restype = ctypes.c_char_p
    lib.ob200_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib, fn, ext


def test_noalloc_entry_point_matches_allocating_entry_point_twice():
    lib, fn, ext = _lib_and_ext()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for m, n in [(300, 517), (129, 64)]:  # second call: smaller shape over the dirty scratch
        L = torch.randn(m, m, device=dev)
        G = torch.randn(m, n, device=dev)
        R = torch.randn(n, n, device=dev)
        P = torch.full((m, n), float("nan"), device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(L.data_ptr(), G.data_ptr(), R.data_ptr(), P.data_ptr(), m, n, stream)
        assert rc == 0, lib.ob200_noalloc_strerror(rc)
        assert torch.cuda.memory_allocated() == before  # nothing taken from torch's allocator
        expected = ext.two_sided_apply(L, G, R)
        torch.cuda.synchronize()
        assert torch.equal(P, expected)  # same kernels, same order of operations
        ref = (L.double() @ G.double() @ R.double()).float()
        assert torch.allclose(P, ref, rtol=1e-4, atol=1e-2)


def test_noalloc_entry_point_rejects_oversized_and_bad_arguments():
    lib, fn, _ = _lib_and_ext()
    dev = torch.device("cuda")
    x = torch.zeros(4, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    m, n = 2048, 1024  # 2 Mi elements > 1 Mi
    assert m * n > MAX_ELEMS
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), m, n, stream)
    assert rc == -2 and b"exceeds" in lib.ob200_noalloc_strerror(rc)
    assert fn(None, x.data_ptr(), x.data_ptr(), x.data_ptr(), 2, 2, stream) == -1
    assert fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, 2, stream) == -1
    torch.cuda.synchronize()
