"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they need a kernel (for example
while a stream is being captured, or inside an application that forbids allocation after start-up),
so the library offers one variant whose scratch lives inside the library image.  This test calls it
the way such a caller would — raw device pointers through ctypes, no torch op involved in the call —
and checks it against the regular entry point on two consecutive calls (the scratch is shared and
keeps the previous call's contents, so the second call is the one that would expose stale data).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from dataflow_b200.ops import native
    lib = ctypes.CDLL(native().__file__)
    fn = lib.dfb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.dfb_noalloc_strerror.restype = ctypes.c_char_p
    lib.dfb_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    from dataflow_b200.ops import resolve_kernels
    K = resolve_kernels()
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, cols) in enumerate([(1000, 4096), (333, 1024)]):
        torch.manual_seed(call)
        x = torch.randn(rows, cols, device="cuda").bfloat16()
        dy = torch.randn(rows, cols, device="cuda").bfloat16()
        w = (torch.randn(cols, device="cuda") + 1).bfloat16()
        _, rstd = K.rmsnorm_fwd(x, w, 1e-5)
        dw_ref = torch.zeros(cols, device="cuda", dtype=torch.bfloat16)
        dx_ref = K.rmsnorm_bwd(dy, x, w, rstd, dw=dw_ref, accumulate=False)
        dx = torch.full_like(x, float("nan"))
        dw = torch.full((cols,), float("nan"), device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = lib.dfb_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                         dw.data_ptr(), rows, cols, stream)
        assert rc == 0, lib.dfb_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert _rel(dx, dx_ref) < 5e-3 and _rel(dw, dw_ref) < 1e-2
        assert torch.equal(dx, dx_ref) and torch.equal(dw, dw_ref)      # same kernels, same order: same bytes


def test_noalloc_rejects_unsupported_sizes():
    lib = _lib()
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    assert lib.dfb_rmsnorm_bwd_noalloc(p, p, p, p, p, p, 4, 8200, None) == -1      # wider than the built-in scratch
    assert lib.dfb_rmsnorm_bwd_noalloc(p, p, p, p, p, p, 4, 100, None) == -1       # not a multiple of 8
    assert lib.dfb_rmsnorm_bwd_noalloc(None, p, p, p, p, p, 4, 64, None) == -2
    assert b"8192" in lib.dfb_noalloc_strerror(-1)
    # a pointer into the middle of a 16-byte vector is refused before anything launches
    assert lib.dfb_rmsnorm_bwd_noalloc(p + 2, p, p, p, p, p, 4, 64, None) == -4
    assert lib.dfb_rmsnorm_bwd_noalloc(p, p, p, p + 2, p, p, 4, 64, None) == -4
    assert b"aligned" in lib.dfb_noalloc_strerror(-4)
